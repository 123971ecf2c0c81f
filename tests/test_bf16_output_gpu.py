"""Dense float formats with the accumulator rounded to bfloat16 on the way out
("<format>.bf16", `gemm(..., out_dtype=torch.bfloat16)`): an output variant of
this build, checked against the oracle's float32 product to one bfloat16 ulp."""

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
