"""Output variants this build adds to the reference's GEMM: dense float formats
with the accumulator rounded to bfloat16 or IEEE half on the way out
("<format>.bf16" / "<format>.f16", `gemm(..., out_dtype=)`), checked against
the oracle's float32 product to one unit in the last place of the output
type; an output scale factor (`gemm(..., alpha=)`, og_b200_launch_alpha),
checked against the oracle's product times alpha; and a per-column bias
(`gemm(..., bias=)`, og_b200_launch_bias), checked against alpha x product +
bias computed from the oracle's float32 product."""

import numpy as np
import pytest
import torch

import opengemm_b200 as og
from opengemm_b200 import capi
from opengemm_b200.configs import heuristic_config
from oracle import opengemm_oracle as ora
from tests.gemm_util import make_case, oracle_of, to_device

pytestmark = pytest.mark.gpu

PLANS = [
    None,                                   # what gemm() would pick
    dict(use_2cta=True, output_n=256),
    dict(use_2cta=False, output_n=96),      # a width that is not a whole number of 64-column staging rows
    dict(use_2cta=False, output_n=64, swap_ab=True),  # transposed stores
    dict(use_2cta=True, output_n=128, epi_direct=1),  # each thread its own row
]


def run(case, name, config):
    m, n, k = case["m"], case["n"], case["k"]
    d = og.dtypes.lookup(name)
    lib, g = capi.bind(name, m, n, k, config)
    out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    out.view(torch.uint8).fill_(0x7F)
    lib.set_wait_limit_ms(1000)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.launch_checked(g, to_device(case["a"], d.a), to_device(case["b"], d.b), None, None, out, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("base", ["bf16", "tf32", "e4m3", "e4m3xe5m2", "e2m1", "e3m2"])
@pytest.mark.parametrize("shape", [(300, 520, 768), (2304, 2560, 1024), (77, 33, 128)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("plan", PLANS, ids=lambda p: "default" if p is None else "-".join(f"{k}{int(v)}" for k, v in p.items()))
def test_bf16_output_is_the_rounded_f32_product(base, shape, plan):
    m, n, k = shape
    case = make_case(base, m, n, k, seed=21)
    config = heuristic_config(base, m, n, k)
    if plan:
        config.update(plan, cluster_m=2 if plan.get("use_2cta") else 1)
    got = run(case, base + ".bf16", config)
    ok, worst = ora.check_bf16_output(got, oracle_of(case))
    assert ok, f"{base}.bf16 {m}x{n}x{k}: {worst:.2f} bfloat16 ulps from the float32 product"


def test_gemm_takes_out_dtype_and_a_bfloat16_out():
    case = make_case("e4m3", 256, 384, 512, seed=3)
    a, b = to_device(case["a"], torch.float8_e4m3fn), to_device(case["b"], torch.float8_e4m3fn)
    want = oracle_of(case)
    c = og.gemm(a, b, out_dtype=torch.bfloat16)
    assert c.dtype is torch.bfloat16 and c.shape == (256, 384)
    into = torch.empty((256, 384), device="cuda", dtype=torch.bfloat16)
    assert og.gemm(a, b, out=into) is into
    torch.cuda.synchronize()
    for t in (c, into):
        ok, worst = ora.check_bf16_output(t.view(torch.int16).cpu().numpy().view(np.uint16), want)
        assert ok, worst
    with pytest.raises(TypeError):
        og.gemm(a.view(torch.int8), b.view(torch.int8), out_dtype=torch.bfloat16)  # integer formats keep int32


def _scaled_case(name, m, n, k, config, alpha, bf16_out=False):
    """Run one GEMM with an output scale; returns (output as numpy, float32 reference x alpha)."""
    case = make_case(name, m, n, k, seed=33)
    d = og.dtypes.lookup(name + (".bf16" if bf16_out else ""))
    lib, g = capi.bind(name + (".bf16" if bf16_out else ""), m, n, k, config)
    scaled = d.impl == "smm"
    out = torch.empty((m, n), device="cuda", dtype=d.out)
    out.view(torch.uint8).fill_(0x7F)
    lib.launch_alpha(g, to_device(case["a"], d.a), to_device(case["b"], d.b),
                     to_device(case["sfa"], d.sf) if scaled else None, to_device(case["sfb"], d.sf) if scaled else None,
                     out, alpha)
    torch.cuda.synchronize()
    fa = ora.dequantize(name, case["a"], case.get("sfa_raw"), k, "a").astype(np.float32)
    fb = ora.dequantize(name, case["b"], case.get("sfb_raw"), k, "b").astype(np.float32)
    want = (fa @ fb.T).astype(np.float32) * np.float32(alpha)
    if d.out is torch.bfloat16:
        return out.view(torch.int16).cpu().numpy().view(np.uint16), want
    return out.cpu().numpy(), want


@pytest.mark.parametrize("alpha", [0.125, 1.0 / 3.0, -2.5])
@pytest.mark.parametrize("name,shape,knobs", [
    ("e4m3", (300, 520, 768), {}),
    ("bf16", (2304, 2560, 1024), dict(use_2cta=True, output_n=256)),   # TMA-store epilogue, several tiles per CTA
    ("tf32", (77, 33, 128), {}),
    ("e4m3", (64, 2048, 512), dict(swap_ab=True, use_2cta=False, output_n=64)),  # transposed stores
    ("bf16", (2304, 2560, 1024), dict(use_2cta=True, output_n=128, split_k=2)),  # stream-K: scaled once, by the finisher
], ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else None)
def test_alpha_scales_float32_output(name, shape, knobs, alpha):
    m, n, k = shape
    config = heuristic_config(name, m, n, k)
    config.update(knobs, cluster_m=2 if knobs.get("use_2cta", config["use_2cta"]) else 1)
    got, want = _scaled_case(name, m, n, k, config, alpha)
    ok, figure = ora.check_north_star(name, got, want)
    assert ok, f"{name} {m}x{n}x{k} alpha={alpha}: {figure}"


@pytest.mark.parametrize("name,bf16_out,knobs", [
    ("nvfp4", False, dict(use_2cta=True, output_n=256)),   # single accumulator: scaled output takes the general loop
    ("mxfp8", False, dict(use_2cta=False, output_n=128)),
    ("e4m3", True, dict(use_2cta=True, output_n=192)),
])
def test_alpha_scales_bfloat16_output(name, bf16_out, knobs):
    m, n, k = 2304, 2568, 1024
    config = heuristic_config(name, m, n, k)
    config.update(knobs, cluster_m=2 if knobs["use_2cta"] else 1)
    got, want = _scaled_case(name, m, n, k, config, 0.3125, bf16_out)
    ok, worst = ora.check_bf16_output(got, want)
    assert ok, f"{name} alpha: {worst:.2f} bfloat16 ulps"


def test_alpha_through_gemm_and_refusal_for_integers():
    case = make_case("e4m3", 256, 384, 512, seed=3)
    a, b = to_device(case["a"], torch.float8_e4m3fn), to_device(case["b"], torch.float8_e4m3fn)
    c = og.gemm(a, b, alpha=0.5)
    torch.cuda.synchronize()
    ok, figure = ora.check_north_star("e4m3", c.cpu().numpy(), oracle_of(case) * np.float32(0.5))
    assert ok, figure
    i8 = torch.ones((128, 128), device="cuda", dtype=torch.int8)
    with pytest.raises(TypeError):
        og.gemm(i8, i8, alpha=2.0)
    lib, g = capi.bind("s8", 128, 128, 128, heuristic_config("s8", 128, 128, 128))
    with pytest.raises(RuntimeError, match="cannot be scaled"):
        lib.launch_alpha(g, i8, i8, None, None, torch.empty((128, 128), device="cuda", dtype=torch.int32), 2.0)


def _half_run(case, name, config):
    m, n, k = case["m"], case["n"], case["k"]
    d = og.dtypes.lookup(name)
    lib, g = capi.bind(name, m, n, k, config)
    out = torch.empty((m, n), device="cuda", dtype=torch.float16)
    out.view(torch.uint8).fill_(0x7B)  # 0x7b7b is a large finite half
    lib.launch(g, to_device(case["a"], d.a), to_device(case["b"], d.b), None, None, out)
    torch.cuda.synchronize()
    return out.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("base", ["bf16", "f16", "tf32", "e4m3", "e2m3"])
@pytest.mark.parametrize("shape", [(300, 520, 768), (2304, 2560, 1024), (77, 33, 128)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("plan", PLANS, ids=lambda p: "default" if p is None else "-".join(f"{k}{int(v)}" for k, v in p.items()))
def test_f16_output_is_the_rounded_f32_product(base, shape, plan):
    m, n, k = shape
    case = make_case(base, m, n, k, seed=22)
    config = heuristic_config(base, m, n, k)
    if plan:
        config.update(plan, cluster_m=2 if plan.get("use_2cta") else 1)
    got = _half_run(case, base + ".f16", config)
    ok, worst = ora.check_f16_output(got, oracle_of(case))
    assert ok, f"{base}.f16 {m}x{n}x{k}: {worst:.2f} half ulps from the float32 product"


def test_gemm_takes_a_float16_out_dtype():
    case = make_case("bf16", 256, 384, 512, seed=4)
    a, b = to_device(case["a"], torch.bfloat16), to_device(case["b"], torch.bfloat16)
    c = og.gemm(a, b, out_dtype=torch.float16)
    assert c.dtype is torch.float16 and c.shape == (256, 384)
    torch.cuda.synchronize()
    ok, worst = ora.check_f16_output(c.view(torch.int16).cpu().numpy().view(np.uint16), oracle_of(case))
    assert ok, worst


def _biased_case(name, m, n, k, config, alpha, variant=""):
    """One GEMM with alpha and a per-column bias; returns (output as numpy, alpha x product + bias in float32)."""
    case = make_case(name, m, n, k, seed=44)
    d = og.dtypes.lookup(name + variant)
    lib, g = capi.bind(name + variant, m, n, k, config)
    scaled = d.impl == "smm"
    rng = np.random.default_rng(9)
    bias = (rng.standard_normal(n) * 3).astype(np.float32)
    out = torch.empty((m, n), device="cuda", dtype=d.out)
    out.view(torch.uint8).fill_(0x7B)
    lib.launch_bias(g, to_device(case["a"], d.a), to_device(case["b"], d.b),
                    to_device(case["sfa"], d.sf) if scaled else None, to_device(case["sfb"], d.sf) if scaled else None,
                    out, alpha, torch.from_numpy(bias).cuda())
    torch.cuda.synchronize()
    fa = ora.dequantize(name, case["a"], case.get("sfa_raw"), k, "a").astype(np.float32)
    fb = ora.dequantize(name, case["b"], case.get("sfb_raw"), k, "b").astype(np.float32)
    want = (fa @ fb.T).astype(np.float32) * np.float32(alpha) + bias[None, :]
    if d.out in (torch.bfloat16, torch.float16):
        return out.view(torch.int16).cpu().numpy().view(np.uint16), want
    return out.cpu().numpy(), want


@pytest.mark.parametrize("alpha", [1.0, -0.75])
@pytest.mark.parametrize("name,shape,knobs", [
    ("e4m3", (300, 520, 768), {}),
    ("bf16", (2304, 2560, 1024), dict(use_2cta=True, output_n=256)),   # TMA-store epilogue, several tiles per CTA
    ("tf32", (77, 33, 128), {}),
    ("e4m3", (64, 2048, 512), dict(swap_ab=True, use_2cta=False, output_n=64)),  # transposed stores: bias rides the MMA rows
    ("bf16", (300, 520, 768), dict(use_2cta=False, output_n=96, epi_direct=1)),  # each thread its own row
    ("bf16", (2304, 2560, 1024), dict(use_2cta=True, output_n=128, split_k=2)),  # stream-K: added once, by the finisher
], ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else None)
def test_bias_is_added_to_float32_output(name, shape, knobs, alpha):
    m, n, k = shape
    config = heuristic_config(name, m, n, k)
    config.update(knobs, cluster_m=2 if knobs.get("use_2cta", config["use_2cta"]) else 1)
    got, want = _biased_case(name, m, n, k, config, alpha)
    ok, figure = ora.check_north_star(name, got, want)
    assert ok, f"{name} {m}x{n}x{k} alpha={alpha} + bias: {figure}"


@pytest.mark.parametrize("name,variant,knobs", [
    ("nvfp4", "", dict(use_2cta=True, output_n=256)),   # single accumulator: biased output takes the general loop
    ("mxfp4", "", dict(use_2cta=False, output_n=128)),
    ("e4m3", ".bf16", dict(use_2cta=True, output_n=192)),
    ("bf16", ".f16", dict(use_2cta=True, output_n=256)),
])
def test_bias_is_added_to_two_byte_output(name, variant, knobs):
    m, n, k = 2304, 2568, 1024
    config = heuristic_config(name, m, n, k)
    config.update(knobs, cluster_m=2 if knobs["use_2cta"] else 1)
    got, want = _biased_case(name, m, n, k, config, 0.5, variant)
    ok, worst = (ora.check_f16_output if variant == ".f16" else ora.check_bf16_output)(got, want)
    assert ok, f"{name}{variant} bias: {worst:.2f} ulps"


def test_bias_through_gemm_and_its_refusals():
    case = make_case("e4m3", 256, 384, 512, seed=3)
    a, b = to_device(case["a"], torch.float8_e4m3fn), to_device(case["b"], torch.float8_e4m3fn)
    bias = torch.linspace(-4, 4, 384, device="cuda")
    c = og.gemm(a, b, bias=bias, alpha=0.25)
    torch.cuda.synchronize()
    want = oracle_of(case) * np.float32(0.25) + bias.cpu().numpy()[None, :]
    ok, figure = ora.check_north_star("e4m3", c.cpu().numpy(), want)
    assert ok, figure
    with pytest.raises(TypeError, match="bias must be"):
        og.gemm(a, b, bias=bias[:100])
    i8 = torch.ones((128, 128), device="cuda", dtype=torch.int8)
    with pytest.raises(TypeError):
        og.gemm(i8, i8, bias=torch.zeros(128, device="cuda"))


@pytest.mark.parametrize("out_format", ["nvfp4", "mxfp8", "mxfp4"])
@pytest.mark.parametrize("name,shape,knobs", [
    ("nvfp4", (300, 512, 768), dict(use_2cta=False, output_n=128)),
    ("nvfp4", (2304, 2560, 1024), dict(use_2cta=True, output_n=256)),   # single accumulator
    ("mxfp8", (1000, 1024, 512), dict(use_2cta=True, output_n=192)),
    ("e4m3", (77, 192, 256), dict(use_2cta=False, output_n=64)),        # a dense format through its bfloat16-output kernel
    ("bf16", (2304, 2560, 1024), dict(use_2cta=True, output_n=128, split_k=2)),  # stream-K: quantised once, by the finisher
], ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else None)
def test_block_scaled_output_equals_quantising_the_bfloat16_product(name, shape, knobs, out_format):
    """C written block-scaled by the epilogue (og_b200_launch_quantized) against
    the same GEMM written as bfloat16 and then quantised by the oracle's
    restatement of the reference's quantize + to_blocked: the same bytes."""
    m, n, k = shape
    case = make_case(name, m, n, k, seed=55)
    base = og.dtypes.lookup(name)
    scaled = base.impl == "smm"
    kernel_name = name if scaled else name + ".bf16"
    d = og.dtypes.lookup(kernel_name)
    config = heuristic_config(name, m, n, k)
    config.update(knobs, swap_ab=False, cluster_m=2 if knobs["use_2cta"] else 1)
    lib, g = capi.bind(kernel_name, m, n, k, config)
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    sfa = to_device(case["sfa"], d.sf) if scaled else None
    sfb = to_device(case["sfb"], d.sf) if scaled else None
    plain = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    lib.launch(g, a, b, sfa, sfb, plain)
    target = og.DTYPES[out_format]
    packed = torch.full((m, n // 2 if target.bits == 4 else n), 0x7B, device="cuda", dtype=torch.uint8)
    block = 16 if out_format == "nvfp4" else 32
    scale_bytes = (-(-m // 128) * 128) * (-(-(n // block) // 4) * 4)
    scales = torch.zeros(scale_bytes, device="cuda", dtype=torch.uint8)
    lib.launch_quantized(g, a, b, sfa, sfb, packed, scales, out_format)
    torch.cuda.synchronize()
    c = ora.bf16_to_f32(plain.view(torch.int16).cpu().numpy().view(np.uint16))
    want_packed, want_scales = ora.quantize(c, out_format)
    assert np.array_equal(packed.cpu().numpy(), np.asarray(want_packed).view(np.uint8).reshape(m, -1))
    assert np.array_equal(scales.cpu().numpy(), ora.to_blocked(want_scales))


def test_block_scaled_output_through_gemm_feeds_the_next_gemm():
    """gemm(..., out_format=) hands back operands the next block-scaled gemm() takes as they are."""
    m, n, k, n2 = 256, 512, 1024, 384
    first = make_case("nvfp4", m, n, k, seed=61)
    second = make_case("nvfp4", n2, n2, n, seed=62)  # only its B operand (n2 x n) is used
    d = og.DTYPES["nvfp4"]
    a, b = to_device(first["a"], d.a), to_device(first["b"], d.b)
    sfa, sfb = to_device(first["sfa"], d.sf), to_device(first["sfb"], d.sf)
    packed, scales = og.gemm(a, b, sfa, sfb, out_format="nvfp4")
    assert packed.dtype is d.a and packed.shape == (m, n // 2) and scales.dtype is d.sf
    b2, sfb2 = to_device(second["b"], d.b), to_device(second["sfb"], d.sf)
    chained = og.gemm(packed, b2, scales, sfb2)
    torch.cuda.synchronize()
    # the oracle's view of the chain: quantise the oracle-checked bfloat16 C, then the second product
    c = og.gemm(a, b, sfa, sfb)
    torch.cuda.synchronize()
    qc, qs = ora.quantize(ora.bf16_to_f32(c.view(torch.int16).cpu().numpy().view(np.uint16)), "nvfp4")
    want = ora.reference("nvfp4", np.asarray(qc).view(np.uint8).reshape(m, -1), second["b"], qs, second["sfb_raw"])
    got = chained.view(torch.int16).cpu().numpy().view(np.uint16)
    ok, worst = ora.check_close("nvfp4", n, got, want)
    assert ok, worst
    ok, figure = ora.check_north_star("nvfp4", got, want)
    assert ok, figure
    with pytest.raises(ValueError, match="multiple of 64"):
        og.gemm(a, to_device(first["b"][:200], d.b), sfa, sfb, out_format="nvfp4")
    i8 = torch.ones((128, 128), device="cuda", dtype=torch.int8)
    with pytest.raises(TypeError):
        og.gemm(i8, i8, out_format="mxfp8")
