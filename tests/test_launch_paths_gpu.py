"""The host side of a launch: the remembered parameter blocks and the prepared
launch must never hand a kernel another call's parameters.  Every call below
differs from the one before it in exactly one thing a parameter block depends
on (an operand address, the output address, alpha, the status word, the bound
configuration, the wait limit), reuses addresses the library has seen, and is
checked against the CPU oracle."""

import numpy as np
import pytest
import torch

from opengemm_b200 import capi
from opengemm_b200.dtypes import lookup
from tests.gemm_util import assert_parity, make_case, oracle_of, to_device

pytestmark = pytest.mark.gpu

M, N, K = 200, 328, 256


def device_case(name, seed):
    case = make_case(name, M, N, K, seed=seed)
    d = lookup(name)
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    sfa = to_device(case["sfa"], d.sf) if d.impl == "smm" else None
    sfb = to_device(case["sfb"], d.sf) if d.impl == "smm" else None
    return case, d, a, b, sfa, sfb


def host(out, d):
    return out.view(torch.int16).cpu().numpy().view(np.uint16) if d.out is torch.bfloat16 else out.cpu().numpy()


@pytest.mark.parametrize("name", ["bf16", "s8", "nvfp4"])
def test_remembered_parameters_follow_every_input(name):
    one, d, a1, b1, sfa1, sfb1 = device_case(name, seed=41)
    two, _, a2, b2, sfa2, sfb2 = device_case(name, seed=42)
    lib, g = capi.bind(name, M, N, K, dict(use_2cta=False, output_n=64))
    out = torch.empty((M, N), device="cuda", dtype=d.out)

    def run(a, b, sfa, sfb, case, into=out, bound=g):
        into.view(torch.uint8).fill_(0x7F)
        lib.launch(bound, a, b, sfa, sfb, into)
        torch.cuda.synchronize()
        assert_parity(case, host(into, d))

    for _ in range(2):  # the second pass finds every block remembered
        run(a1, b1, sfa1, sfb1, one)
        run(a2, b2, sfa2, sfb2, two)  # same output address, other operands
    mixed = dict(one, b=two["b"])
    if "sfb_raw" in two:
        mixed.update(sfb=two["sfb"], sfb_raw=two["sfb_raw"])
    run(a1, b2, sfa1, sfb2, mixed)  # one operand swapped under a remembered output address
    other = torch.empty((M, N), device="cuda", dtype=d.out)
    run(a1, b1, sfa1, sfb1, one, into=other)
    # another configuration for the same shape and buffers: another plan, other tensor maps
    lib2, g2 = capi.bind(name, M, N, K, dict(use_2cta=True, output_n=128, cluster_m=2))
    run(a1, b1, sfa1, sfb1, one, bound=g2)
    run(a1, b1, sfa1, sfb1, one)
    # a status word and a wait limit change the block too
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out.view(torch.uint8).fill_(0x7F)
    lib.launch_checked(g, a1, b1, sfa1, sfb1, out, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_parity(one, host(out, d))
    lib.set_wait_limit_ms(500)
    try:
        run(a1, b1, sfa1, sfb1, one)
    finally:
        lib.set_wait_limit_ms(2000)


def test_alpha_is_part_of_what_is_remembered():
    case, d, a, b, _, _ = device_case("bf16", seed=43)
    lib, g = capi.bind("bf16", M, N, K, dict(use_2cta=False, output_n=64))
    out = torch.empty((M, N), device="cuda", dtype=torch.float32)
    want = oracle_of(case)
    for alpha in (0.5, 0.5, -2.0, 1.0):
        lib.launch_alpha(g, a, b, None, None, out, alpha)
        torch.cuda.synchronize()
        np.testing.assert_allclose(out.cpu().numpy(), alpha * want, rtol=1e-3, atol=1e-3 * np.abs(want).max())
    lib.launch(g, a, b, None, None, out)
    torch.cuda.synchronize()
    assert_parity(case, out.cpu().numpy())


@pytest.mark.parametrize("name", ["bf16", "mxfp8"])
def test_prepared_launch_equals_launch(name):
    case, d, a, b, sfa, sfb = device_case(name, seed=44)
    lib, g = capi.bind(name, M, N, K, dict(use_2cta=False, output_n=64))
    plain = torch.empty((M, N), device="cuda", dtype=d.out)
    prepared = torch.empty((M, N), device="cuda", dtype=d.out)
    lib.launch(g, a, b, sfa, sfb, plain)
    step = lib.launcher(g, a, b, sfa, sfb, prepared)
    for _ in range(3):
        prepared.view(torch.uint8).fill_(0x7F)
        step()
        torch.cuda.synchronize()
        assert torch.equal(plain.view(torch.uint8), prepared.view(torch.uint8))
    assert_parity(case, host(prepared, d))
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):  # the stream is looked up at call time
        prepared.view(torch.uint8).fill_(0x7F)
        step()
    side.synchronize()
    assert torch.equal(plain.view(torch.uint8), prepared.view(torch.uint8))
