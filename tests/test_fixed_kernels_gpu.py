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
    ("e4m3xe5m2.bf16", dict(use_2cta=True, output_n=256), 1024),
    ("nvfp4", dict(use_2cta=True, output_n=192), 1024),
    ("nvfp4", dict(use_2cta=True, output_n=256), 1024),
    ("mxfp4", dict(use_2cta=True, output_n=256), 1024),
    ("mxfp4", dict(use_2cta=False, output_n=256), 2048),
    ("mxfp8", dict(use_2cta=True, output_n=256), 1024),
    ("mxfp8", dict(use_2cta=True, output_n=192), 1024),
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
