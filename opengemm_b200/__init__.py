"""opengemm_b200: GEMM kernels for NVIDIA B200 (sm_100a) behind OpenGEMM's interface.

    import opengemm_b200 as og
    c = og.gemm(a, b)                      # dense
    c = og.gemm(a, b, sfa, sfb)            # block-scaled
    og.emit_kernel(a, b, file="k.cu")      # a standalone .cu/.cuh pair
    og.run_kernel("k.cu", a, b)            # compile and run it

The public names are those of the reference package (opengemm/__init__.py:10-28).
Additions of this build, all optional: `og.gemm(..., out_dtype=torch.bfloat16)`
and `og.gemm(..., alpha=0.5)` (output variants), `og.quantize_blocked` (values ->
packed data + blocked scales in one kernel), `python -m opengemm_b200.tune`
and `python -m opengemm_b200.benchmark` (tuner and suite runner).
"""

from .api import gemm
from .build import prebuild
from .dtypes import DTYPES, dtype_name
from .emit import emit_kernel
from .quant import pack, quantize, quantize_blocked, to_blocked, unpack
from .run import run_kernel

__all__ = [
    "gemm",
    "prebuild",
    "emit_kernel",
    "run_kernel",
    "dtype_name",
    "DTYPES",
    "quantize",
    "to_blocked",
    "pack",
    "unpack",
]
__version__ = "0.1.4+b200"
