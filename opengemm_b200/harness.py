"""Seeded inputs, the torch reference product, tolerances, library baselines and
CUDA-event timing shared by the tuner and the command-line tools.

The contract follows the reference's harness module
(opengemm/python/bench.py:20-295): uniform [-1, 1) operands (full-range
integers for s8/u8, tf32 pre-rounded, sub-byte formats packed, block-scaled
formats quantised from bf16), an fp32 / exact-integer reference with TF32 off,
`(rtol, atol)` growing with sqrt(K / 4096), input rotations larger than twice
L2, and medians of CUDA-event windows around back-to-back launches.
"""

import datetime
import itertools
import os
import statistics
from typing import NamedTuple

import torch

from .dtypes import DTYPES, elems, k_of, sf_block
from .quant import SMALL_FLOATS, pack, quantize, round_tf32, to_blocked, unpack

# (rtol, atol) at K = 4096
TOLERANCE = {"s8": (0.0, 0.0), "u8": (0.0, 0.0), "nvfp4": (2.0**-6, 2.0**-5), "mxfp8": (2.0**-6, 2.0**-5),
             "mxfp4": (2.0**-6, 2.0**-5)}
DEFAULT_TOLERANCE = (1.0e-3, 2.0e-2)
INT_RANGE = {"s8": (-127, 128), "u8": (0, 256)}


class Inputs(NamedTuple):
    """One rotation of operands and the output buffer the kernel writes."""

    a: torch.Tensor
    b: torch.Tensor
    sfa: torch.Tensor = None      # blocked scales, what the kernel reads
    sfb: torch.Tensor = None
    sfa_raw: torch.Tensor = None  # (rows, K / block) scales, what the reference reads
    sfb_raw: torch.Tensor = None
    out: torch.Tensor = None


def tolerance(name, k):
    rtol, atol = TOLERANCE.get(name, DEFAULT_TOLERANCE)
    grow = max(1.0, (k / 4096) ** 0.5)
    return rtol * grow, atol * grow


def make_inputs(m, n, k, name, seed=0, device="cuda"):
    """Operands for one GEMM, seeded; different seeds give different rotations."""
    d = DTYPES[name]
    g = torch.Generator(device=device).manual_seed(seed)
    if d.out is torch.int32:
        lo, hi = INT_RANGE[name]
        draw = lambda rows: torch.randint(lo, hi, (rows, k), generator=g, device=device, dtype=torch.int32)
        return Inputs(draw(m).to(d.a).contiguous(), draw(n).to(d.b).contiguous())
    a = torch.rand((m, k), generator=g, device=device) * 2 - 1
    b = torch.rand((n, k), generator=g, device=device) * 2 - 1
    if d.impl == "smm":
        qa, sfa = quantize(a.to(torch.bfloat16), name)
        qb, sfb = quantize(b.to(torch.bfloat16), name)
        return Inputs(qa, qb, to_blocked(sfa), to_blocked(sfb), sfa, sfb)
    if name == "tf32":
        return Inputs(round_tf32(a), round_tf32(b))
    if d.bits < 8:
        return Inputs(pack(a, name), pack(b, name))
    return Inputs(a.to(d.a).contiguous(), b.to(d.b).contiguous())


def iteration_bytes(name, m, n, k):
    """Bytes one GEMM must move (operands, scales, output once each)."""
    d = DTYPES[name]
    nbytes = (m * k + n * k) * d.bits // 8 + m * n * d.out.itemsize
    if d.impl == "smm":
        nbytes += (m * k + n * k) // sf_block(d)
    return nbytes


def make_input_set(m, n, k, name, seed=0, cap_bytes=16 << 30):
    """Enough rotations to exceed twice L2, each with its own output."""
    per = iteration_bytes(name, m, n, k)
    l2 = torch.cuda.get_device_properties(torch.cuda.current_device()).L2_cache_size
    count = max(2, min(-(-2 * l2 // per), cap_bytes // per))
    sets = []
    for i in range(count):
        one = make_inputs(m, n, k, name, seed + i)
        sets.append(one._replace(out=torch.empty((m, n), device="cuda", dtype=DTYPES[name].out)))
    return sets


def _values(t, elem, k):
    return unpack(t.view(torch.uint8), elem, k) if elem in SMALL_FLOATS else t.float()


def reference(entry, name):
    """The product the kernel is checked against: fp32 of the upcast (or
    dequantised) operands, exact for the integer formats; on whatever device
    the operands live."""
    d = DTYPES[name]
    before = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        k = k_of(d, entry.a.size(1))
        if d.out is torch.int32:
            return torch.mm(entry.a.double(), entry.b.double().t()).to(torch.int32)
        if d.impl == "smm":
            elem, block = elems(name)[0], sf_block(d)
            a = _values(entry.a, elem, k) * entry.sfa_raw.float().repeat_interleave(block, dim=1)
            b = _values(entry.b, elem, k) * entry.sfb_raw.float().repeat_interleave(block, dim=1)
            return (a @ b.t()).to(torch.bfloat16)
        ea, eb = elems(name)
        return torch.mm(_values(entry.a, ea, k), _values(entry.b, eb, k).t()).to(d.out)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = before


def runner(buffers, bound):
    """A zero-argument callable launching the bound kernel on the next rotation."""
    lib, g = bound
    if hasattr(lib, "launcher"):  # addresses taken once per rotation, not once per call
        cycle = itertools.cycle([(lib.launcher(g, r.a, r.b, r.sfa, r.sfb, r.out), r.out) for r in buffers])

        def call():
            launch, out = next(cycle)
            launch()
            return out

        return call
    cycle = itertools.cycle(buffers)

    def call():
        r = next(cycle)
        lib.launch(g, r.a, r.b, r.sfa, r.sfb, r.out)
        return r.out

    return call


def correctness_error(buffers, bound, name, k, want=None):
    """None when the bound kernel reproduces the reference on the first
    rotation, else the first line of the mismatch."""
    rtol, atol = tolerance(name, k)
    try:
        out = runner(buffers[:1], bound)()
        torch.cuda.synchronize()
        torch.testing.assert_close(out, reference(buffers[0], name) if want is None else want, rtol=rtol, atol=atol)
        return None
    except Exception as exc:
        return str(exc).splitlines()[0][:90]


def baseline_for(buffers, name):
    """torch's library kernel for this format over the same rotations, or
    `(None, reason)` where it has none."""
    d = DTYPES[name]
    r0 = buffers[0]
    one = torch.ones((), device="cuda", dtype=torch.float32)
    if name in ("bf16", "f16"):
        cycle = itertools.cycle([(r.a, r.b.t(), r.out) for r in buffers])
        call = lambda: (lambda a, b, c: torch.mm(a, b, out=c, out_dtype=d.out))(*next(cycle))
    elif name == "s8":
        cycle = itertools.cycle([(r.a, r.b.t(), r.out) for r in buffers])
        call = lambda: (lambda a, b, c: torch._int_mm(a, b, out=c))(*next(cycle))
    elif name in ("e4m3", "e4m3xe5m2"):
        cycle = itertools.cycle([(r.a, r.b.t(), r.out) for r in buffers])
        call = lambda: (lambda a, b, c: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=d.out, out=c))(*next(cycle))
    elif name in ("nvfp4", "mxfp8"):
        cycle = itertools.cycle([(r.a, r.b.t(), r.sfa, r.sfb, r.out) for r in buffers])
        call = lambda: (lambda a, b, sa, sb, c: torch._scaled_mm(a, b, sa, sb, out_dtype=torch.bfloat16, out=c))(*next(cycle))
    else:
        return None, f"torch has no library kernel for {name}"
    try:
        call()
        torch.cuda.synchronize()
        return call, None
    except Exception as exc:
        return None, str(exc).splitlines()[0][:110]


def elapsed_us(fn, iterations):
    """Microseconds per call over `iterations` back-to-back calls, by CUDA events."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iterations):
        fn()
    end.record()
    end.synchronize()
    return start.elapsed_time(end) * 1e3 / iterations


def timed(fn, window_ms=20.0, repeats=3, warmup=3, max_iterations=4000):
    """Median microseconds per call over `repeats` windows of about `window_ms`."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    guess = max(elapsed_us(fn, 5), 0.5)
    iterations = int(max(5, min(max_iterations, window_ms * 1e3 / guess)))
    return statistics.median(elapsed_us(fn, iterations) for _ in range(repeats))


def env_stamp():
    return {"gpu": torch.cuda.get_device_name(0), "device": os.environ.get("CUDA_VISIBLE_DEVICES", "unpinned"),
            "torch": torch.__version__, "date": datetime.date.today().isoformat()}
