"""C[M, N] = A[M, K] @ B[N, K].T on B200: the user-facing `gemm`.

Same contract as the reference's `gemm` (opengemm/python/api.py:66-90):
operands are contiguous 2-D CUDA tensors with K innermost, the output is a
new or caller-supplied row-major tensor (float32; int32 for s8/u8; bfloat16
for block-scaled formats), the launch is asynchronous on the current stream
of the operands' device, and validation raises the same TypeError /
ValueError texts (api.py:25-63).
"""

import torch

from . import capi
from .configs import resolve_config
from .dtypes import DTYPES, NARROW_OUT, NARROW_OUT_SUFFIXES, base_name, dtype_name, extent, k_of, lookup, sf_block

_bound = {}  # (dtype name, m, n, k, launch mode) -> (Library, OgGemm), for the life of the process


def bind(name, m, n, k, device):
    """Resolve and memoise the kernel for a shape in the library's current launch mode."""
    with torch.cuda.device(device):
        config = resolve_config(base_name(name), m, n, k)  # the bf16-output variant runs its format's tile plan
    _bound[(name, m, n, k, capi.independent_inputs())] = capi.bind(name, m, n, k, config)
    return _bound[(name, m, n, k, capi.independent_inputs())]


def forget(name=None):
    """Drop memoised bindings (after the stored configurations changed)."""
    for key in [key for key in _bound if name is None or base_name(key[0]) == name]:
        del _bound[key]


def scale_bytes(d, rows, k):
    """Bytes of a scale tensor in the 128x4 blocked layout."""
    return (-(-rows // 128) * 128) * (-(-k // (sf_block(d) * 4)) * 4)


def check_operands(d, m, n, k, a, b, sfa, sfb):
    """Raise unless the operands are what a kernel for this format and shape reads."""
    cols = extent(d, k)
    for label, t, rows, want in (("a", a, m, d.a), ("b", b, n, d.b)):
        if not (t.is_cuda and t.dim() == 2 and t.is_contiguous()):
            raise TypeError(f"{label} must be a contiguous 2-D CUDA tensor")
        if t.dtype is not want or t.shape != (rows, cols):
            raise TypeError(f"{label} must be {want} [{rows}, {cols}], got {t.dtype} {list(t.shape)}")
    if b.device != a.device:
        raise ValueError(f"a is on {a.device} and b on {b.device}")
    if d.impl == "mm":
        if sfa is not None or sfb is not None:
            raise TypeError("a dense format takes no scales")
        return
    if sfa is None or sfb is None:
        raise TypeError("a block-scaled format takes both sfa and sfb")
    for label, t, rows in (("sfa", sfa, m), ("sfb", sfb, n)):
        if not (t.is_cuda and t.is_contiguous() and t.dtype is d.sf and t.device == a.device):
            raise TypeError(
                f"{label} must be a contiguous {d.sf} tensor on {a.device}, in the 128x4 blocked layout"
            )
        want = scale_bytes(d, rows, k)
        if t.numel() < want:
            raise ValueError(
                f"{label} must hold {want} bytes of the 128x4 blocked scale layout, got {t.numel()}"
            )


def output(d, m, n, out, device):
    """The tensor C is written to: `out` after checks, or a new row-major one."""
    if out is None:
        return torch.empty((m, n), device=device, dtype=d.out)
    if not (out.is_contiguous() and out.shape == (m, n) and out.dtype is d.out and out.device == device):
        raise ValueError(f"out must be a contiguous {d.out} [{m}, {n}] on {device}")
    if out.data_ptr() % 16:
        raise ValueError("out must start on a 16-byte boundary")
    return out


def gemm(a, b, sfa=None, sfb=None, out=None, atype=None, btype=None, out_dtype=None, alpha=None, bias=None,
         out_format=None):
    """Compute C[M, N] = A[M, K] @ B[N, K].T.

    Args:
        a: `(M, K)` operand.
        b: `(N, K)` operand.
        sfa: scales of `a` in the 128x4 blocked layout (`to_blocked` builds it);
            block-scaled formats only.
        sfb: scales of `b`, likewise.
        out: output to write into instead of allocating one.
        atype: element name for a `uint8` operand: "u8", "e3m2", "e2m3" or "e2m1".
        btype: element name for `b`; defaults to `atype` when the dtypes match.
        out_dtype: `torch.bfloat16` or `torch.float16` makes a dense float
            format round its f32 accumulator to that type on the way out (an
            addition of this build; the default, None, is the reference's
            output type).  Implied by an `out` of that dtype.
        alpha: a Python float every output is multiplied by (in float32) before
            it is stored, e.g. the product of per-tensor scales of fp8 operands
            (an addition of this build; float formats only).
        bias: a float32 CUDA vector of N values added to every row of C (after
            `alpha`, in float32, before the store; an addition of this build;
            float formats only).
        out_format: "nvfp4", "mxfp8" or "mxfp4" makes C leave block-scaled
            along N, bit for bit what `quantize(c.to(bfloat16), out_format)`
            and `to_blocked` would give, ready to be the `a` of the next
            block-scaled GEMM (an addition of this build; float formats only,
            N a multiple of 64).  Returns `(packed, blocked scales)`.

    Returns:
        `(M, N)` row-major: float32 for dense formats (bfloat16 with
        `out_dtype=torch.bfloat16`, float16 with `out_dtype=torch.float16`), int32
        for s8 and u8, bfloat16 for block-scaled ones.
    """
    name = dtype_name(a, b, sfa, atype, btype)
    if out_format is not None:
        return _gemm_quantized(name, a, b, sfa, sfb, out_format)
    if out_dtype is None and out is not None and out.dtype in NARROW_OUT_SUFFIXES and DTYPES[name].out is torch.float32:
        out_dtype = out.dtype
    if out_dtype is not None and out_dtype is not DTYPES[name].out:
        suffix = NARROW_OUT_SUFFIXES.get(out_dtype)
        if suffix is None or name + suffix not in NARROW_OUT:
            raise TypeError(f"{name} writes {DTYPES[name].out}; only dense float formats can write "
                            f"torch.bfloat16 or torch.float16 instead")
        name += suffix
    d = lookup(name)
    m, n, k = a.size(0), b.size(0), k_of(d, a.size(1))
    check_operands(d, m, n, k, a, b, sfa, sfb)
    lib, g = _bound.get((name, m, n, k, capi.independent_inputs())) or bind(name, m, n, k, a.device)
    out = output(d, m, n, out, a.device)
    if alpha is None and bias is None:
        lib.launch(g, a, b, sfa, sfb, out)
        return out
    if d.out is torch.int32:
        raise TypeError(f"{name} accumulates integers exactly: its output cannot be scaled or biased")
    if bias is None:
        lib.launch_alpha(g, a, b, sfa, sfb, out, alpha)
        return out
    if not (bias.is_cuda and bias.device == a.device and bias.dtype is torch.float32 and bias.is_contiguous()
            and bias.shape == (n,)):
        raise TypeError(f"bias must be a contiguous float32 [{n}] on {a.device}")
    lib.launch_bias(g, a, b, sfa, sfb, out, 1.0 if alpha is None else alpha, bias)
    return out


def _gemm_quantized(name, a, b, sfa, sfb, out_format):
    """gemm() with a block-scaled C: `(packed, blocked scales)`."""
    if out_format not in ("nvfp4", "mxfp8", "mxfp4"):
        raise TypeError(f"out_format must be 'nvfp4', 'mxfp8' or 'mxfp4', got {out_format!r}")
    if DTYPES[name].out is torch.int32:
        raise TypeError(f"{name} accumulates integers: its output cannot be block-scaled")
    if DTYPES[name].impl == "mm":
        name += NARROW_OUT_SUFFIXES[torch.bfloat16]  # the kernels that round the accumulator to bfloat16
    d, target = lookup(name), DTYPES[out_format]
    m, n, k = a.size(0), b.size(0), k_of(d, a.size(1))
    check_operands(d, m, n, k, a, b, sfa, sfb)
    if n % 64:
        raise ValueError(f"a block-scaled output needs N to be a multiple of 64, got {n}")
    lib, g = _bound.get((name, m, n, k, "quantized")) or _bind_quantized(name, m, n, k, a.device)
    packed = torch.empty((m, extent(target, n)), device=a.device, dtype=target.a)
    scales = torch.zeros(scale_bytes(target, m, n), device=a.device, dtype=torch.uint8).view(target.sf)
    lib.launch_quantized(g, a, b, sfa, sfb, packed, scales, out_format)
    return packed, scales


def _bind_quantized(name, m, n, k, device):
    """The stored configuration, kept off the operand swap and on 64-column tile multiples."""
    with torch.cuda.device(device):
        config = dict(resolve_config(base_name(name), m, n, k))
    if config.get("swap_ab"):
        config.update(swap_ab=False, use_2cta=m > 128, cluster_m=2 if m > 128 else 1, output_n=128)
    config["output_n"] = max(64, -(-int(config["output_n"]) // 64) * 64) if config["output_n"] % 64 else config["output_n"]
    config["output_n"] = min(config["output_n"], 256)
    _bound[(name, m, n, k, "quantized")] = capi.bind(name, m, n, k, config)
    return _bound[(name, m, n, k, "quantized")]
