"""Compile and run a kernel `emit_kernel` wrote (opengemm/python/run.py:17-68):
nvcc builds `<stem>.so` beside the source (reused while newer than the source
and header), ctypes loads it, the operands go through the same checks as
`gemm`, and the entry point is called on the current stream."""

import ctypes
import subprocess
import time
from pathlib import Path

from .api import check_operands, output
from .build import nvcc_path
from .capi import raw_stream
from .dtypes import DTYPES
from .emit import parse_tag
from .log import log

# The command line the emitted file names in its own header comment.
NVCC_LINE = ["-O3", "-std=c++20", "-gencode=arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr", "-shared",
             "-Xcompiler", "-fPIC"]
_loaded = {}


def build(source):
    """Compile `source` to a shared library beside it unless a current one exists."""
    source = Path(source).resolve()
    header, library = source.with_suffix(".cuh"), source.with_suffix(".so")
    newest = max(p.stat().st_mtime for p in (source, header) if p.exists())
    if library.exists() and library.stat().st_mtime >= newest:
        return library
    started = time.perf_counter()
    done = subprocess.run([nvcc_path(), *NVCC_LINE, str(source), "-o", str(library), "-lcuda"],
                          capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + (done.stderr or done.stdout))
    log(f"built {library.name} in {time.perf_counter() - started:.1f} s")
    return library


def entry_point(source):
    """`(callable, impl, dtype, m, n, k)` for an emitted source; compiled and
    loaded on first use and again when the file changes."""
    path = Path(source)
    if path.suffix != ".cu":
        path = Path(str(path) + ".cu")
    path = path.resolve()
    stamp = path.stat().st_mtime
    hit = _loaded.get(str(path))
    if hit and hit[0] == stamp:
        return hit[1]
    impl, dtype, m, n, k, entry = parse_tag(path.read_text())
    function = getattr(ctypes.CDLL(str(build(path))), entry)
    function.argtypes = [ctypes.c_void_p] * (4 if impl == "mm" else 6)
    function.restype = None
    _loaded[str(path)] = (stamp, (function, impl, dtype, m, n, k))
    return _loaded[str(path)][1]


def run_kernel(file, a, b, sfa=None, sfb=None, out=None):
    """Run the kernel emitted to `file` on these tensors, on the current CUDA stream.

    Args:
        file: the `.cu` path `emit_kernel` wrote (the stem works too).
        a, b: operands in the dtype and shape the kernel was emitted for.
        sfa, sfb: blocked scales; block-scaled kernels only.
        out: row-major output to write into.

    Returns:
        `(M, N)` row-major: float32 or int32 for dense, bfloat16 for block-scaled.
    """
    call, impl, name, m, n, k = entry_point(file)
    d = DTYPES[name]
    check_operands(d, m, n, k, a, b, sfa, sfb)
    out = output(d, m, n, out, a.device)
    operands = (a, b, sfa, sfb, out) if impl == "smm" else (a, b, out)
    call(*(t.data_ptr() for t in operands), ctypes.c_void_p(raw_stream(a.get_device())))
    return out
