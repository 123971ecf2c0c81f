"""Cluster-K (OgGemm.cluster_k with one-CTA MMAs): 2, 4 or 8 CTAs of a
thread-block cluster share every output tile along K and reduce through the
first CTA's shared memory.  On the CPU: the plan lowers a request to what
fits and sizes the grid in whole clusters.  On the GPU: the product equals
the oracle's for every way count, for tiles reused by a persistent cluster
(the landing zone's hand-shake), ragged edges, rows past M, transposed
stores, integer (bit-exact), block-scaled and 2-byte outputs."""

import pytest

from opengemm_b200 import capi
from tests.gemm_util import assert_parity, make_case, run_library


def plan_of(name, m, n, k, **knobs):
    config = dict({"use_2cta": False, "output_n": 64, "swap_ab": False, "epi_direct": 0, "supergroup": 4}, **knobs)
    lib, g = capi.bind(name, m, n, k, config)
    return lib.plan(g)


def test_plan_lowers_the_request_to_what_fits():
    assert plan_of("bf16", 256, 512, 4096, cluster_k=4)["cluster_k"] == 4
    assert plan_of("bf16", 256, 512, 4096, cluster_k=4)["grid"] == 16 * 4             # 2 x 8 tiles, each a cluster of four
    assert plan_of("bf16", 256, 512, 4096, cluster_k=3)["cluster_k"] == 2              # powers of two
    assert plan_of("bf16", 256, 512, 128, cluster_k=8)["cluster_k"] == 2               # two K blocks: two ways at most
    assert plan_of("bf16", 256, 512, 4096, cluster_k=8, output_n=256)["cluster_k"] < 8  # the landing zone must leave a ring
    assert plan_of("bf16", 256, 512, 4096, cluster_k=4, use_2cta=True)["cluster_k"] == 1  # pairs do not split K
    assert plan_of("bf16", 256, 512, 4096, cluster_k=4, split_k=2)["cluster_k"] == 1      # nor does stream-K
    big = plan_of("bf16", 8192, 8192, 4096, cluster_k=4)
    assert big["grid"] == 148 // 4 * 4 and big["fixed_shape"] == 0


CASES = [
    ("bf16", (300, 520, 1024), dict(output_n=64), 2),
    ("bf16", (300, 520, 1024), dict(output_n=64), 4),
    ("bf16", (128, 160, 2048), dict(output_n=32), 8),
    ("s8", (1100, 2100, 2048), dict(output_n=64), 4),            # 9 x 33 tiles on 37 clusters: eight tiles per cluster
    ("e4m3", (64, 2048, 4096), dict(output_n=64, swap_ab=True), 4),   # small M on the N side, transposed stores
    ("tf32", (77, 33, 512), dict(output_n=48), 2),
    ("nvfp4", (64, 1024, 4096), dict(output_n=64), 4),            # rows 64..127 of every tile lie past M
    ("mxfp4", (64, 7168, 8192), dict(output_n=64, swap_ab=True), 2),  # the decode shard
    ("mxfp8", (200, 300 * 2, 1024), dict(output_n=128), 2),
    ("e4m3.bf16", (300, 520, 1024), dict(output_n=64), 4),
]


@pytest.mark.gpu
@pytest.mark.parametrize("name,shape,knobs,ways", CASES,
                         ids=[f"{n}-{'x'.join(map(str, s))}-{w}way" for n, s, _, w in CASES])
def test_cluster_k_matches_the_oracle(name, shape, knobs, ways):
    m, n, k = shape
    base = name.split(".")[0]
    case = make_case(base, m, n, k, seed=31)
    config = dict({"use_2cta": False, "swap_ab": False, "epi_direct": 0, "supergroup": 4, "cluster_k": ways}, **knobs)
    lib, g = capi.bind(name, m, n, k, config)
    assert lib.plan(g)["cluster_k"] == ways
    if name.endswith(".bf16"):
        import numpy as np
        import torch

        from opengemm_b200.dtypes import lookup
        from oracle import opengemm_oracle as ora
        from tests.gemm_util import oracle_of, to_device

        d = lookup(name)
        out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
        out.view(torch.uint8).fill_(0x7F)
        lib.launch(g, to_device(case["a"], d.a), to_device(case["b"], d.b), None, None, out)
        torch.cuda.synchronize()
        ok, worst = ora.check_bf16_output(out.view(torch.int16).cpu().numpy().view(np.uint16), oracle_of(case))
        assert ok, worst
        return
    case["name"] = name
    assert_parity(case, run_library(case, config))


@pytest.mark.gpu
def test_cluster_k_with_bias_and_alpha_is_applied_once_by_the_first_rank():
    import numpy as np
    import torch

    from opengemm_b200.dtypes import DTYPES
    from oracle import opengemm_oracle as ora
    from tests.gemm_util import oracle_of, to_device

    name, (m, n, k) = "bf16", (300, 520, 2048)
    case = make_case(name, m, n, k, seed=32)
    d = DTYPES[name]
    lib, g = capi.bind(name, m, n, k, {"use_2cta": False, "output_n": 64, "cluster_k": 4})
    bias = torch.linspace(-3, 3, n, device="cuda")
    out = torch.empty((m, n), device="cuda", dtype=torch.float32)
    lib.launch_bias(g, to_device(case["a"], d.a), to_device(case["b"], d.b), None, None, out, -0.5, bias)
    torch.cuda.synchronize()
    want = oracle_of(case) * np.float32(-0.5) + bias.cpu().numpy()[None, :]
    ok, figure = ora.check_north_star(name, out.cpu().numpy(), want)
    assert ok, figure
