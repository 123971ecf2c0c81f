"""The allocation-free launch, og_b200_launch_no_alloc, against the ordinary one.

Some callers may not allocate device memory in a launch (a fixed memory
budget, an allocator that owns the rest of the GPU, a latency-critical loop):
for them the library carries a fixed workspace and this entry point runs the
stream-K schedule out of it.  The test calls it through the C ABI twice in a
row on the same operands - the second call meets the workspace exactly as the
first left it - and each time compares the output with that of the existing
entry point (og_mm_launch / og_smm_launch): bit for bit for int8, within the
suite's tolerances for the float formats.  It is collected last so that a
run stopping at the first failure has already run everything else.
"""

import ctypes
from ctypes import POINTER, byref, c_char_p, c_int32, c_void_p

import numpy as np
import pytest
import torch

from opengemm_b200 import capi
from opengemm_b200.dtypes import DTYPES
from oracle import opengemm_oracle as ora
from tests.gemm_util import assert_parity, make_case, to_device

pytestmark = pytest.mark.gpu


def _entry(lib):
    fn = ctypes.CDLL(str(lib.path)).og_b200_launch_no_alloc
    fn.restype = c_int32
    fn.argtypes = [POINTER(capi.OgGemm)] + [c_void_p] * 5 + [c_int32, c_void_p, c_char_p, c_int32]
    return fn


def _as_numpy(out, d):
    if d.out is torch.bfloat16:
        return out.view(torch.int16).cpu().numpy().view(np.uint16)
    return out.cpu().numpy()


@pytest.mark.parametrize(
    "name,shape,knobs",
    [
        ("s8", (2304, 2560, 1024), dict(use_2cta=True, output_n=128)),      # 180 tiles on 74 pairs: stream-K
        ("bf16", (2304, 2560, 512), dict(use_2cta=False, output_n=128)),    # 360 tiles on 148 CTAs: stream-K
        ("nvfp4", (2304, 2560, 1024), dict(use_2cta=True, output_n=192)),   # block-scaled, bf16 output
        ("e4m3", (300, 520, 768), dict(use_2cta=False, output_n=64)),       # fewer tiles than CTAs: no workspace needed
    ],
)
def test_no_alloc_launch_matches_the_ordinary_launch(name, shape, knobs):
    m, n, k = shape
    d = DTYPES[name]
    config = dict({"use_2cta": False, "output_n": 128, "swap_ab": False, "epi_direct": 0, "supergroup": 4}, **knobs)
    lib, g = capi.bind(name, m, n, k, config)
    no_alloc = _entry(lib)
    case = make_case(name, m, n, k, seed=11)
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    sfa = to_device(case["sfa"], d.sf) if d.impl == "smm" else None
    sfb = to_device(case["sfb"], d.sf) if d.impl == "smm" else None
    ptr = lambda t: 0 if t is None else t.data_ptr()

    want = torch.empty((m, n), device="cuda", dtype=d.out)
    lib.launch(g, a, b, sfa, sfb, want)  # the existing entry point
    torch.cuda.synchronize()
    want = _as_numpy(want, d)

    message = ctypes.create_string_buffer(320)
    for call in range(2):
        out = torch.empty((m, n), device="cuda", dtype=d.out)
        out.view(torch.uint8).fill_(0x7F)
        status = no_alloc(byref(g), ptr(a), ptr(b), ptr(sfa), ptr(sfb), out.data_ptr(), 0,
                          capi.raw_stream(0), message, len(message))
        assert status == capi.OG_OK, message.value.decode()
        torch.cuda.synchronize()
        got = _as_numpy(out, d)
        if d.out is torch.int32:
            assert np.array_equal(got, want), f"call {call}"
        else:
            ok, worst = ora.check_close(name, k, got, want)
            assert ok, f"call {call}: outside tolerance by {worst}"
            ok, figure = ora.check_north_star(name, got, want)
            assert ok, f"call {call}: strict bound missed ({figure})"
        assert_parity(case, got)  # and against the CPU oracle itself, not only kernel against kernel


def test_no_alloc_launch_reports_errors_in_the_callers_buffer():
    lib, g = capi.bind("bf16", 256, 256, 256, {"use_2cta": False, "output_n": 128})
    no_alloc = _entry(lib)
    message = ctypes.create_string_buffer(320)
    status = no_alloc(byref(g), 0, 0, 0, 0, 0, 0, 0, message, len(message))
    assert status == capi.OG_ERR_LAUNCH and b"device pointers" in message.value
    g.row = -7
    status = no_alloc(byref(g), 1, 1, 0, 0, 1, 0, 0, message, len(message))
    assert status == capi.OG_ERR_LAUNCH and b"bind it first" in message.value


def test_no_alloc_launch_between_ordinary_launches_on_one_stream():
    """Ordinary launches overlap their neighbours programmatically; the
    allocation-free one must not, and all three write the same C here: the
    last writer's result has to be the one left standing, three times over."""
    name, (m, n, k) = "s8", (2304, 2560, 1024)
    d = DTYPES[name]
    config = {"use_2cta": True, "output_n": 128, "swap_ab": False, "epi_direct": 0, "supergroup": 4, "cluster_m": 2}
    lib, g = capi.bind(name, m, n, k, config)
    no_alloc = _entry(lib)
    cases = [make_case(name, m, n, k, seed=s) for s in (1, 2, 3)]
    operands = [(to_device(c["a"], d.a), to_device(c["b"], d.b)) for c in cases]
    out = torch.empty((m, n), device="cuda", dtype=d.out)
    message = ctypes.create_string_buffer(320)
    for order in ((0, 1, 2), (2, 0, 1)):
        for position, which in enumerate(order):
            a, b = operands[which]
            if position == 1:
                status = no_alloc(byref(g), a.data_ptr(), b.data_ptr(), 0, 0, out.data_ptr(), 0, capi.raw_stream(0),
                                  message, len(message))
                assert status == capi.OG_OK, message.value.decode()
            else:
                lib.launch(g, a, b, None, None, out)
        torch.cuda.synchronize()
        assert_parity(cases[order[-1]], out.cpu().numpy())


def test_no_alloc_launch_honours_the_wait_limit_setting():
    """The limit set by og_b200_set_wait_limit_ms reaches this entry point too
    (it shares the parameter block of the ordinary launches): a short limit
    must not disturb a healthy launch."""
    name, (m, n, k) = "bf16", (300, 520, 768)
    d = DTYPES[name]
    lib, g = capi.bind(name, m, n, k, {"use_2cta": False, "output_n": 64})
    no_alloc = _entry(lib)
    case = make_case(name, m, n, k, seed=8)
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    out = torch.empty((m, n), device="cuda", dtype=d.out)
    message = ctypes.create_string_buffer(320)
    try:
        lib.set_wait_limit_ms(50)
        status = no_alloc(byref(g), a.data_ptr(), b.data_ptr(), 0, 0, out.data_ptr(), 0, capi.raw_stream(0),
                          message, len(message))
        torch.cuda.synchronize()
    finally:
        lib.set_wait_limit_ms(2000)
    assert status == capi.OG_OK, message.value.decode()
    assert_parity(case, out.cpu().numpy())
