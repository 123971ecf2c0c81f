"""The bounded-wait path, made to run out on purpose in the only way that
faults nothing: a one-CTA launch whose stage barriers are told to expect more
bytes than their loads deliver (og_b200_test_overcredit_next_launch), with
the wait limit set to a few milliseconds.  The MMA role's first wait for data
gives up, raises the CTA's abort flag and writes (site | cta << 8) to the
launch's status word; every role leaves through the ordinary teardown
(tensor memory freed, nothing left spinning), so the context stays usable -
an ordinary launch right after must still be correct.  og_b200_status turns
the word into OG_ERR_TIMEOUT with a readable message."""

import pytest
import torch

from opengemm_b200 import capi
from tests.gemm_util import assert_parity, make_case, run_library, to_device

pytestmark = pytest.mark.gpu

SITE_MMA_FULL = 2


@pytest.mark.parametrize("name,config", [
    ("bf16", {"use_2cta": False, "output_n": 64}),
    ("nvfp4", {"use_2cta": False, "output_n": 64}),
    ("e4m3", {"use_2cta": True, "output_n": 64, "cluster_m": 2}),  # a pair: both CTAs give up and meet in the teardown
])
def test_a_wait_that_runs_out_reports_its_site_and_leaves_the_context_usable(name, config):
    m, n, k = (256 if config["use_2cta"] else 128), 64, 512
    case = make_case(name, m, n, k, seed=5)
    d = capi.lookup(name)
    lib, g = capi.bind(name, m, n, k, config)
    assert lib.plan(g)["grid"] == (2 if config["use_2cta"] else 1)
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    sfa = to_device(case["sfa"], d.sf) if d.impl == "smm" else None
    sfb = to_device(case["sfb"], d.sf) if d.impl == "smm" else None
    out = torch.zeros((m, n), device="cuda", dtype=d.out)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    try:
        lib.set_wait_limit_ms(5)
        lib.test_overcredit_next_launch(16)
        lib.launch_checked(g, a, b, sfa, sfb, out, status)
        torch.cuda.synchronize()  # returns: the kernel ended by itself
    finally:
        lib.set_wait_limit_ms(2000)
    word = int(status.item())
    assert word & 0xFF == SITE_MMA_FULL and word >> 8 == 0, f"status word {word:#x}"
    assert lib.status(word) == capi.OG_ERR_TIMEOUT
    assert "MMA waiting for a stage" in lib.error() and "CTA 0" in lib.error()
    assert lib.status(0) == capi.OG_OK
    # the hook is one-shot and the context is intact: the same launch now runs and is right
    got = run_library(case, config)
    assert_parity(case, got)
