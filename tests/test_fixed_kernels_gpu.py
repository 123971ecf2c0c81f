"""The kernels compiled for one tile shape each (csrc/kernels_fixed_*.cu)
against the run-time-planned kernel they stand in for: the same launch through
the C ABI with og_b200_set_fixed_kernels on and off must give the same bits,
and those must match the CPU oracle.  Shapes are ragged on both sides so the
folded constants meet partial tiles, and several tiles per CTA."""

import numpy as np
import pytest
import torch

from opengemm_b200 import capi
from opengemm_b200.dtypes import lookup
from tests.gemm_util import assert_parity, make_case, oracle_of, to_device
from oracle import opengemm_oracle as ora

FIXED = [
    ("bf16", dict(use_2cta=True, output_n=256), 768),
    ("f16", dict(use_2cta=True, output_n=128), 768),
    ("tf32", dict(use_2cta=True, output_n=256), 512),
    ("s8", dict(use_2cta=True, output_n=256), 1536),
    ("u8", dict(use_2cta=True, output_n=256), 1024),
    ("e4m3", dict(use_2cta=True, output_n=256), 1536),
    ("e2m1", dict(use_2cta=True, output_n=256), 1024),
    # 16-bit output: more than 16 K blocks, below which the plan stores by TMA and no fixed-shape kernel does
    ("e4m3xe5m2.bf16", dict(use_2cta=True, output_n=256), 2304),
    ("nvfp4", dict(use_2cta=True, output_n=192), 4608),
    ("nvfp4", dict(use_2cta=True, output_n=256), 4608),
    ("mxfp4", dict(use_2cta=True, output_n=256), 4608),
    ("mxfp4", dict(use_2cta=False, output_n=256), 4608),
    ("mxfp8", dict(use_2cta=True, output_n=256), 2304),
    ("mxfp8", dict(use_2cta=True, output_n=192), 2304),
]
IDS = [f"{name}-{'pair' if knobs['use_2cta'] else 'single'}-{knobs['output_n']}" for name, knobs, _ in FIXED]


def test_plans_report_which_launches_a_fixed_shape_kernel_serves():
    for name, knobs, k in FIXED:
        config = dict({"swap_ab": False, "epi_direct": 0, "supergroup": 4, "cluster_m": 2 if knobs["use_2cta"] else 1}, **knobs)
        lib, g = capi.bind(name, 2400, 1000, k, config)
        assert lib.plan(g)["fixed_shape"] == 1, (name, knobs)
        for off in (dict(use_clc=True), dict(walk=1), dict(stages=3), dict(swap_ab=True), dict(epi_direct=1),
                    dict(output_n=64)):
            lib, g = capi.bind(name, 2400, 1000, k, dict(config, **off))
            assert lib.plan(g)["fixed_shape"] == 0, (name, off)


@pytest.mark.gpu
@pytest.mark.parametrize("name,knobs,k", FIXED, ids=IDS)
def test_fixed_shape_kernel_equals_the_run_time_kernel(name, knobs, k):
    m, n = 2400, 1000
    base = name.split(".")[0]
    case = make_case(base, m, n, k, seed=23)
    d = lookup(name)
    config = dict({"swap_ab": False, "epi_direct": 0, "supergroup": 4, "cluster_m": 2 if knobs["use_2cta"] else 1}, **knobs)
    lib, g = capi.bind(name, m, n, k, config)
    assert lib.plan(g)["fixed_shape"] == 1
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    sfa = to_device(case["sfa"], d.sf) if d.impl == "smm" else None
    sfb = to_device(case["sfb"], d.sf) if d.impl == "smm" else None
    outs = []
    try:
        for fixed in (True, False):
            lib.set_fixed_kernels(fixed)
            out = torch.empty((m, n), device="cuda", dtype=d.out)
            out.view(torch.uint8).fill_(0x7F)
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            lib.launch_checked(g, a, b, sfa, sfb, out, status)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            outs.append(out)
    finally:
        lib.set_fixed_kernels(True)
    assert torch.equal(outs[0].view(torch.uint8), outs[1].view(torch.uint8))
    if d.out is torch.bfloat16:
        got = outs[0].view(torch.int16).cpu().numpy().view(np.uint16)
    else:
        got = outs[0].cpu().numpy()
    if name.endswith(".bf16"):
        ok, worst = ora.check_bf16_output(got, oracle_of(case))
        assert ok, worst
    else:
        assert_parity(case, got)


# The feature-free build of every variant (csrc/kernels_plain_*.cu): one small
# ragged shape per format and tile arrangement, so that every store path of the
# epilogue (own row, staged rows, transposed) is met.
PLAIN = [
    (name, knobs)
    for name in ("bf16", "f16", "tf32", "s8", "u8", "e4m3", "e5m2", "e3m2", "e2m3", "e2m1", "e4m3xe5m2",
                 "bf16.bf16", "tf32.bf16", "e4m3.bf16", "nvfp4", "mxfp8", "mxfp4")
    for knobs in (dict(use_2cta=False, output_n=64, swap_ab=False, epi_direct=0),
                  dict(use_2cta=False, output_n=32, swap_ab=True, epi_direct=1),
                  dict(use_2cta=True, output_n=128, swap_ab=False, epi_direct=1))
]
PLAIN_IDS = [f"{name}-{'pair' if k['use_2cta'] else 'single'}-{k['output_n']}{'-swap' if k['swap_ab'] else ''}" for name, k in PLAIN]


def test_plans_report_which_launches_the_feature_free_kernel_serves():
    for name, knobs in PLAIN:
        config = dict({"supergroup": 4, "cluster_m": 2 if knobs["use_2cta"] else 1}, **knobs)
        lib, g = capi.bind(name, 300, 520, 768, config)
        plan = lib.plan(g)
        assert plan["plain"] == 1 and plan["fixed_shape"] == 0, (name, knobs, plan)
        for off in (dict(use_clc=True), dict(walk=1), dict(walk=3)):
            lib, g = capi.bind(name, 300, 520, 768, dict(config, **off))
            assert lib.plan(g)["plain"] == 0, (name, off)
    lib, g = capi.bind("bf16", 64, 8192, 8192, dict(use_2cta=False, output_n=128, cluster_k=4))
    assert lib.plan(g)["plain"] == 0 and lib.plan(g)["cluster_k"] > 1
    lib, g = capi.bind("bf16.f16", 300, 520, 768, dict(use_2cta=False, output_n=64))
    assert lib.plan(g)["plain"] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name,knobs", PLAIN, ids=PLAIN_IDS)
def test_feature_free_kernel_equals_the_full_kernel(name, knobs):
    m, n, k = 300, 520, 768
    base = name.split(".")[0]
    case = make_case(base, m, n, k, seed=29)
    d = lookup(name)
    config = dict({"supergroup": 4, "cluster_m": 2 if knobs["use_2cta"] else 1}, **knobs)
    lib, g = capi.bind(name, m, n, k, config)
    assert lib.plan(g)["plain"] == 1
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    sfa = to_device(case["sfa"], d.sf) if d.impl == "smm" else None
    sfb = to_device(case["sfb"], d.sf) if d.impl == "smm" else None
    outs = []
    try:
        for special in (True, False):
            lib.set_fixed_kernels(special)
            out = torch.empty((m, n), device="cuda", dtype=d.out)
            out.view(torch.uint8).fill_(0x7F)
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            lib.launch_checked(g, a, b, sfa, sfb, out, status)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            outs.append(out)
    finally:
        lib.set_fixed_kernels(True)
    assert torch.equal(outs[0].view(torch.uint8), outs[1].view(torch.uint8))
    if d.out is torch.bfloat16:
        got = outs[0].view(torch.int16).cpu().numpy().view(np.uint16)
    else:
        got = outs[0].cpu().numpy()
    if name.endswith(".bf16"):
        ok, worst = ora.check_bf16_output(got, oracle_of(case))
        assert ok, worst
    else:
        assert_parity(case, got)
