"""The baseline's own configurations, each in its own format, at its own size
and in its own value distribution, and every N/2, N/4 and N/8 shard of the
three it shards along N.

Operands come from bench.make_operands (N(0,1) -> bf16; N(0,1)*16 clamped to
+-448 -> e4m3; N(0,1)*64 clamped to +-57344 -> e5m2; s8 uniform over all of
[-128, 127]; nvfp4 with amax/6 ue4m3 scales per 16; mxfp4 with
2^floor(log2(amax/6)) ue8m0 scales per 32).  The configuration is the one
gemm() would run (configs.resolve_config), called through the C ABI into a
sentinel-filled output; the CPU oracle recomputes sampled rows and columns
(bench.sampled_oracle_check): bit-exact for s8, max|x-ref|/max|ref| <= 1e-3
for f32 outputs, 1 bf16 ulp + 1e-2 relative for block-scaled outputs, and the
reference's own assert_close tolerances (scripts/test.py:33-48,
opengemm/python/bench.py:28-35,71-75) in every case.  A shard is the last
rank's: rows shard_bounds(N, g, g-1) of the full B and of its blocked scales,
so the slicing of both is under test as well.
"""

import functools

import pytest
import torch

import bench
from opengemm_b200 import capi, configs, shard
from opengemm_b200.dtypes import DTYPES

pytestmark = pytest.mark.gpu

CASES = [(key, 1) for key in ("c1", "c2", "c2m", "c3", "c4", "c5")]
CASES += [(key, g) for key in bench.SHARDED for g in (2, 4, 8)]


@functools.lru_cache(maxsize=1)
def full_operands(key):
    """The whole configuration's operands; the most recent one is kept so the
    shards of a configuration reuse it."""
    work = bench.WORKLOADS[key]
    torch.cuda.empty_cache()
    return bench.make_operands(torch, work["name"], work["m"], work["n"], work["k"], seed=0, device=torch.device("cuda", 0))


@pytest.mark.parametrize("key,ways", CASES, ids=[f"{k}-1of{g}" if g > 1 else k for k, g in CASES])
def test_baseline_configuration_matches_the_oracle(key, ways):
    work = bench.WORKLOADS[key]
    name, m, n_full, k = work["name"], work["m"], work["n"], work["k"]
    d = DTYPES[name]
    ops = full_operands(key)
    rank = ways - 1
    n0, n1 = shard.shard_bounds(n_full, ways, rank)
    n = n1 - n0
    if ways > 1:
        sfb = None if ops.sfb is None else shard.shard_scales(ops.sfb, name, n_full, k, ways, rank)
        ops = bench.Operands(ops.a, shard.shard_rows(ops.b, ways, rank), ops.sfa, sfb, ops.sfa_raw,
                             None if ops.sfb_raw is None else ops.sfb_raw[n0:n1])
    if name == "s8":
        assert int(ops.a.min()) == -128 and int(ops.b.min()) == -128  # the full range, -128 x -128 included
    # The store may hold one configuration per launch mode (overlapping launches of
    # independent GEMMs, what bench.py times; dependent launches, the library's default):
    # both are what gemm() would run, so both are checked where they differ.
    tried = []
    for dependent in (False, True):
        config = configs.resolve_config(name, m, n, k, dependent=dependent)
        if config in tried:
            continue
        tried.append(config)
        lib, g = capi.bind(name, m, n, k, config)
        out = torch.empty((m, n), device="cuda", dtype=d.out)
        out.view(torch.uint8).fill_(0x7F)
        lib.set_wait_limit_ms(2000)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        lib.launch_checked(g, ops.a, ops.b, ops.sfa, ops.sfb, out, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, f"device wait gave up: {int(status.item())} ({lib.plan(g)})"
        result = bench.sampled_oracle_check(torch, name, k, ops, out)
        print(f"{key} {m}x{n}x{k} {name} ({'dependent' if dependent else 'independent'} launches): {result}")
        assert result["ok"], result
        if d.out is torch.int32:
            assert result["max_rel"] == 0.0
        del out


def test_c3_full_output_has_no_sentinel_left():
    """Every element of a baseline-size output is written (sampled rows cannot show a skipped tile)."""
    work = bench.WORKLOADS["c3"]
    name, m, n, k = work["name"], work["m"], work["n"] // 8, work["k"]
    ops = bench.make_operands(torch, name, m, n, k, seed=3, device=torch.device("cuda", 0))
    lib, g = capi.bind(name, m, n, k, configs.resolve_config(name, m, n, k))
    out = torch.full((m, n), 0x7F7F7F7F, device="cuda", dtype=torch.int32)
    lib.launch(g, ops.a, ops.b, None, None, out)
    torch.cuda.synchronize()
    assert int((out == 0x7F7F7F7F).sum()) == 0  # |sum| <= 8192 * 128^2 = 2^27 < the sentinel
