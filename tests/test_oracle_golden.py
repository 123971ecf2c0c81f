"""The numpy oracle against fixtures produced by the reference's own Python.

The fixtures in tests/golden/ were written by tests/golden/make_golden.py from
`opengemm.python.bench.reference` and `opengemm.python.quant` run on a CPU.
Integer and byte results must match bit for bit; the float32 products may
differ from torch's by summation order only, so they are held to 1e-5 of the
row scale, far inside the reference's own acceptance tolerance.
"""

import numpy as np
import pytest

from oracle import opengemm_oracle as ora

NAMES = list(ora.FORMATS)
SHAPES = [(77, 33, 128), (64, 48, 256), (130, 72, 384)]


def load(golden_dir, name):
    return np.load(golden_dir / f"gemm_{name}.npz")


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_reference_product_matches_golden(golden_dir, name, shape):
    m, n, k = shape
    z = load(golden_dir, name)
    tag = f"{m}x{n}x{k}"
    a, b = z[f"{tag}.a"], z[f"{tag}.b"]
    smm = ora.impl_of(name) == "smm"
    sfa = z[f"{tag}.sfa_raw"] if smm else None
    sfb = z[f"{tag}.sfb_raw"] if smm else None
    got = ora.reference(name, a, b, sfa, sfb)
    want = z[f"{tag}.c"]
    assert got.shape == (m, n)
    out = ora.FORMATS[name][4]
    if out == "s32":
        assert np.array_equal(got, want)
    elif out == "f32":
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= 1e-5 * scale
    else:  # bf16 bits: a float32 sum that lands on a rounding boundary may differ by one ulp
        g, w = ora.as_float(name, got), ora.as_float(name, want)
        assert (np.abs(g - w) <= ora.bf16_ulp(w)).all()
        assert (got == want).mean() > 0.99
    rtol, atol = z[f"{tag}.tol"]
    assert ora.tolerance(name, k) == (rtol, atol)
    ok, _ = ora.check_close(name, k, got, want)
    assert ok
    ok, _ = ora.check_north_star(name, got, want)
    assert ok


@pytest.mark.parametrize("name", ["nvfp4", "mxfp8", "mxfp4"])
def test_blocked_scales_round_trip(golden_dir, name):
    z = load(golden_dir, name)
    for m, n, k in SHAPES:
        tag = f"{m}x{n}x{k}"
        for which, rows in (("sfa", m), ("sfb", n)):
            rawsf = z[f"{tag}.{which}_raw"]
            blocked = z[f"{tag}.{which}"]
            assert np.array_equal(ora.to_blocked(rawsf), blocked)
            assert blocked.size == ora.scale_bytes(name, rows, k)
            assert np.array_equal(ora.from_blocked(blocked, rows, rawsf.shape[1]), rawsf)


def test_small_float_tables_and_packing(golden_dir):
    z = np.load(golden_dir / "quant.npz")
    x = z["x"]
    for elem in ("e3m2", "e2m3", "e2m1"):
        assert np.array_equal(ora.small_float_values(elem), z[f"values.{elem}"])
        assert np.array_equal(ora.pack(x, elem), z[f"pack.{elem}"])
        assert np.array_equal(ora.unpack(z[f"pack.{elem}"], elem, 256), z[f"unpack.{elem}"])
    assert np.array_equal(ora.round_tf32(x), z["round_tf32"])
    assert np.array_equal(ora.to_blocked(z["to_blocked.in"]), z["to_blocked.out"])


@pytest.mark.parametrize("name", ["nvfp4", "mxfp8", "mxfp4"])
@pytest.mark.parametrize("tag", ["randn", "rand"])
def test_quantize_matches_golden(golden_dir, name, tag):
    z = np.load(golden_dir / "quant.npz")
    x = ora.bf16_to_f32(z[f"quantize.{name}.{tag}.in"])
    packed, scales = ora.quantize(x, name)
    assert np.array_equal(scales, z[f"quantize.{name}.{tag}.scales"])
    assert np.array_equal(packed, z[f"quantize.{name}.{tag}.packed"])
    assert np.array_equal(ora.to_blocked(scales), z[f"quantize.{name}.{tag}.blocked"])


def test_fp8_tables_match_torch():
    torch = pytest.importorskip("torch")
    codes = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    for table, dtype in ((ora.E4M3_TABLE, torch.float8_e4m3fn), (ora.E5M2_TABLE, torch.float8_e5m2),
                         (ora.E8M0_TABLE, torch.float8_e8m0fnu)):
        want = codes.view(dtype).float().numpy()
        assert np.array_equal(np.isnan(table), np.isnan(want))
        keep = ~np.isnan(want)
        assert np.array_equal(table[keep], want[keep])
    x = (torch.randn(4096, generator=torch.Generator().manual_seed(3)) * 100).clamp(-448, 448)
    assert np.array_equal(ora.f32_to_e4m3(x.numpy()), x.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    y = (torch.randn(4096, generator=torch.Generator().manual_seed(4)) * 1000).clamp(-57344, 57344)
    assert np.array_equal(ora.f32_to_e5m2(y.numpy()), y.to(torch.float8_e5m2).view(torch.uint8).numpy())
    z = torch.randn(4096, generator=torch.Generator().manual_seed(5)) * 50
    assert np.array_equal(ora.f32_to_bf16(z.numpy()), z.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
