"""GPU parity: the CUDA library, called through its C ABI, against the oracle
and against the golden fixtures produced by the reference's Python.

Shapes are the ragged and aligned ones of the reference's own suite
(scripts/test.py:23-30) plus small fixtures; tolerances are the reference's
(bench.py:28-35) and the stricter bound stated for this build: bit-exact
int32; max|x-ref|/max|ref| <= 1e-3 for f32 outputs; <= 1 bf16 ulp + 1e-2
relative for block-scaled outputs.
"""

import numpy as np
import pytest

from oracle import opengemm_oracle as ora
from tests.gemm_util import assert_parity, golden_case, make_case, run_library

pytestmark = pytest.mark.gpu

NAMES = list(ora.FORMATS)
GOLDEN_SHAPES = [(77, 33, 128), (64, 48, 256), (130, 72, 384)]
# Four of the reference's six test shapes (scripts/test.py:23-30); the two large ones, 2048^3 and 1 x 8192 x 8192,
# run for every format in test_shape_suite_gpu.py, where the oracle recomputes sampled rows and columns instead of
# unpacking whole operands on the CPU.
REFERENCE_SHAPES = [(128, 128, 128), (300, 520, 768), (77, 33, 128), (2048, 2048, 384)]


@pytest.mark.parametrize("name", NAMES)
def test_golden_fixtures(golden_dir, name):
    z = np.load(golden_dir / f"gemm_{name}.npz")
    for m, n, k in GOLDEN_SHAPES:
        case = golden_case(z, name, m, n, k)
        got = run_library(case)
        assert_parity(case, got, want=case["c"])
        assert_parity(case, got)


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("shape", REFERENCE_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_reference_suite_shapes(name, shape):
    m, n, k = shape
    case = make_case(name, m, n, k, seed=0)
    assert_parity(case, run_library(case))


def _config(name, **knobs):
    base = {"use_2cta": False, "output_n": 128, "swap_ab": False, "epi_direct": 0, "supergroup": 4}
    base.update(knobs)
    return base


VARIANTS = [
    dict(use_2cta=False, output_n=128),
    dict(use_2cta=False, output_n=256),
    dict(use_2cta=True, output_n=128),
    dict(use_2cta=True, output_n=256),
    dict(use_2cta=True, output_n=192),
    dict(use_2cta=False, output_n=64),
    dict(use_2cta=True, output_n=64, epi_direct=1),
    dict(use_2cta=False, output_n=128, swap_ab=True),
    dict(use_2cta=True, output_n=64, swap_ab=True),
    dict(use_2cta=False, output_n=128, epi_direct=1, stages=2),
]


@pytest.mark.parametrize("name", ["bf16", "tf32", "s8", "e4m3xe5m2", "e2m1", "e3m2", "nvfp4", "mxfp8", "mxfp4"])
@pytest.mark.parametrize("variant", VARIANTS, ids=lambda v: "-".join(f"{k}{int(v[k])}" for k in v))
def test_tile_plans(name, variant):
    """Every way of tiling the same product must give the same answer: pair or
    single CTA, each tile width, swapped operands, direct or staged epilogue."""
    m, n, k = 520, 712, 1152
    case = make_case(name, m, n, k, seed=1)
    assert_parity(case, run_library(case, _config(name, **variant)))


@pytest.mark.parametrize("name", ["nvfp4", "mxfp8", "mxfp4"])
@pytest.mark.parametrize("two", [True, False], ids=["pair", "single"])
def test_single_accumulator_is_reused_across_tiles(name, two):
    """A 256-wide block-scaled tile has one accumulator in tensor memory; the
    epilogue hands it back before its last stores, and every CTA here computes
    more than one tile, so a hand-back that came too early would corrupt the
    next tile.  N is ragged: the last tile column is clipped by the stores."""
    from opengemm_b200 import capi

    m, n, k = 2304, 2568, 1024
    config = _config(name, use_2cta=two, output_n=256)
    lib, g = capi.bind(name, m, n, k, config)
    plan = lib.plan(g, 0)
    assert plan["acc_slots"] == 1 and plan["tiles"] > plan["grid"] // plan["cta_group"]
    case = make_case(name, m, n, k, seed=9)
    assert_parity(case, run_library(case, config))


STREAM_K_PLANS = [
    dict(use_2cta=True, output_n=128),
    dict(use_2cta=False, output_n=64),
    dict(use_2cta=True, output_n=192),
    dict(use_2cta=True, output_n=256, epi_direct=1),
    dict(use_2cta=False, output_n=64, swap_ab=True),
]


@pytest.mark.parametrize("name", ["bf16", "s8", "e2m1", "nvfp4", "mxfp8", "mxfp4"])
@pytest.mark.parametrize("variant", STREAM_K_PLANS, ids=lambda v: "-".join(f"{k}{int(v[k])}" for k in v))
def test_stream_k_schedule(name, variant):
    """split_k >= 2 deals the (tile, K-block) units out in equal ranges: tiles
    shared by two clusters are summed through the partial-sum workspace.  The
    shape has more tiles than clusters and not a whole number of waves; s8 must
    stay bit-exact."""
    from opengemm_b200 import capi

    m, n, k = 2304, 2560, 1024
    config = _config(name, split_k=2, **variant)
    lib, g = capi.bind(name, m, n, k, config)
    assert lib.plan(g, 0)["stream_k"] == 1
    case = make_case(name, m, n, k, seed=4)
    want = None
    for _ in range(2):  # twice: the second launch meets flags left by the first
        got = run_library(case, config)
        if want is None:
            from tests.gemm_util import oracle_of

            want = oracle_of(case)
        assert_parity(case, got, want=want)


@pytest.mark.parametrize(
    "name,shape,knobs",
    [
        ("bf16", (256, 256, 4096), dict(use_2cta=False, output_n=128)),       # 4 tiles, each cut ~37 ways
        ("s8", (300, 520, 4096), dict(use_2cta=True, output_n=256)),          # 6 ragged tiles over 74 pairs
        ("mxfp4", (64, 7168, 8192), dict(use_2cta=False, output_n=64, swap_ab=True)),   # decode shard: 56 tiles, 148 CTAs
        ("nvfp4", (64, 3072, 2048), dict(use_2cta=False, output_n=64, swap_ab=True)),
        ("mxfp4", (64, 57344, 1024), dict(use_2cta=False, output_n=64, swap_ab=True)),  # 3 whole waves + 4 tiles cut along K
        ("e4m3", (1, 8192, 8192), dict(use_2cta=False, output_n=16, swap_ab=True)),
    ],
)
def test_stream_k_many_way_split(name, shape, knobs):
    """With fewer tiles than clusters (or a small remainder wave) a tile is cut
    along K across many clusters and finished by the one holding its first blocks."""
    from opengemm_b200 import capi

    m, n, k = shape
    config = _config(name, split_k=2, **knobs)
    lib, g = capi.bind(name, m, n, k, config)
    plan = lib.plan(g, 0)
    assert plan["stream_k"] == 1 and plan["grid"] == 148
    case = make_case(name, m, n, k, seed=8)
    for _ in range(2):
        assert_parity(case, run_library(case, config))


@pytest.mark.parametrize("name", ["bf16", "s8", "nvfp4"])
@pytest.mark.parametrize("two", [False, True], ids=["single", "pair"])
@pytest.mark.parametrize("shape", [(520, 712, 1152), (4096, 4096, 512), (3000, 2100, 128)], ids=lambda s: "x".join(map(str, s)))
def test_cluster_launch_control_scheduler(name, two, shape):
    """use_clc: one cluster per tile, running clusters take over the tiles of
    clusters that have not started; the product must not change.  The shapes
    cover fewer tiles than SMs, many more tiles than SMs, and very short K
    loops (the producer runs several tiles ahead of the epilogue)."""
    from opengemm_b200 import capi

    m, n, k = shape
    config = _config(name, use_2cta=two, output_n=128, use_clc=True)
    lib, g = capi.bind(name, m, n, k, config)
    plan = lib.plan(g, 0)
    assert plan["use_clc"] == 1 and plan["grid"] == plan["tiles"] * plan["cta_group"]
    case = make_case(name, m, n, k, seed=9)
    assert_parity(case, run_library(case, config))


@pytest.mark.parametrize("name", ["bf16", "s8", "nvfp4"])
def test_dense_rows_of_ones_known_answer(name):
    """A known-answer case no tolerance is needed for: all-ones operands give K everywhere."""
    m, n, k = 192, 320, 256
    case = make_case(name, m, n, k, seed=2)
    impl = ora.impl_of(name)
    if name == "bf16":
        case["a"] = np.full((m, k), 0x3F80, dtype=np.uint16)
        case["b"] = np.full((n, k), 0x3F80, dtype=np.uint16)
    elif name == "s8":
        case["a"] = np.ones((m, k), dtype=np.int8)
        case["b"] = np.ones((n, k), dtype=np.int8)
    else:
        case["a"] = np.full((m, k // 2), 0x22, dtype=np.uint8)  # e2m1 code 2 = 1.0, twice per byte
        case["b"] = np.full((n, k // 2), 0x22, dtype=np.uint8)
        case["sfa_raw"] = np.full((m, k // 16), 0x38, dtype=np.uint8)  # ue4m3 1.0
        case["sfb_raw"] = np.full((n, k // 16), 0x38, dtype=np.uint8)
        case["sfa"], case["sfb"] = ora.to_blocked(case["sfa_raw"]), ora.to_blocked(case["sfb_raw"])
    got = ora.as_float(name, run_library(case))
    assert (got == float(k)).all(), (impl, np.unique(got)[:8])


def test_large_seeded_s8_is_bit_exact():
    case = make_case("s8", 1024, 2048, 4096, seed=3)
    got = run_library(case)
    assert np.array_equal(got, ora.reference("s8", case["a"], case["b"]))


@pytest.mark.parametrize("name,shape", [("bf16", (300, 520, 768)), ("s8", (1024, 1024, 1024)), ("e3m2", (77, 33, 128)),
                                        ("nvfp4", (300, 520, 768)), ("mxfp4", (16, 2048, 1024))])
def test_emitted_kernel_matches_the_oracle(tmp_path, name, shape):
    """emit_kernel + run_kernel: the standalone artefact computes the same product."""
    import torch

    import opengemm_b200 as og
    from tests.gemm_util import to_device

    m, n, k = shape
    case = make_case(name, m, n, k, seed=6)
    d = og.DTYPES[name]
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    scales = (to_device(case["sfa"], d.sf), to_device(case["sfb"], d.sf)) if d.impl == "smm" else ()
    names = {"atype": name} if d.a is torch.uint8 else {}
    stem = tmp_path / f"{name}_{m}_{n}_{k}"
    og.emit_kernel(a, b, *scales, file=str(stem), **names)
    out = torch.empty((m, n), device="cuda", dtype=d.out)
    out.view(torch.uint8).fill_(0x7F)
    og.run_kernel(str(stem) + ".cu", a, b, *scales, out=out)
    torch.cuda.synchronize()
    got = out.view(torch.int16).cpu().numpy().view(np.uint16) if d.out is torch.bfloat16 else out.cpu().numpy()
    assert_parity(case, got)
