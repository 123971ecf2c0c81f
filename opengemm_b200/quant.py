"""Packing and quantising values into the formats gemm() takes (torch, any device).

Public behaviour follows opengemm/python/quant.py:8-122: `pack` / `unpack` for
the 6- and 4-bit elements (nearest value, a tie to the even code, first value
in the low bits), `quantize` for nvfp4 / mxfp8 / mxfp4, `to_blocked` for the
128x4 scale layout, `round_tf32`.  `pack` here locates the nearest code with a
sorted search instead of scanning all 16 or 64 codes.
"""

import torch

from .dtypes import DTYPES, elems, sf_block

# exponent bits, mantissa bits, storage bits
SMALL_FLOATS = {"e3m2": (3, 2, 6), "e2m3": (2, 3, 6), "e2m1": (2, 1, 4)}


def _values(elem, device):
    """Value of every code of a small float, in code order (sign, exponent, mantissa)."""
    ebits, mbits, _ = SMALL_FLOATS[elem]
    bias = (1 << (ebits - 1)) - 1
    code = torch.arange(1 << (1 + ebits + mbits), dtype=torch.int32)
    sign = 1.0 - 2.0 * (code >> (ebits + mbits)).double()
    e = ((code >> mbits) & ((1 << ebits) - 1)).double()
    f = (code & ((1 << mbits) - 1)).double() / (1 << mbits)
    mag = torch.where(e == 0, f * 2.0 ** (1 - bias), (1 + f) * torch.pow(2.0, e - bias))
    return (sign * mag).float().to(device)


def _pack_bits(codes, bits):
    group = {6: 4, 4: 2}[bits]  # codes per packed word
    nbytes = group * bits // 8
    rows, k = codes.shape
    c = codes.reshape(rows, k // group, group).to(torch.int64)
    shifts = torch.arange(group, device=codes.device, dtype=torch.int64) * bits
    word = (c << shifts).sum(dim=-1)
    byte_shifts = torch.arange(nbytes, device=codes.device, dtype=torch.int64) * 8
    out = (word.unsqueeze(-1) >> byte_shifts) & 0xFF
    return out.reshape(rows, k // group * nbytes).to(torch.uint8).contiguous()


def _unpack_bits(packed, k, bits):
    group = {6: 4, 4: 2}[bits]
    nbytes = group * bits // 8
    rows = packed.shape[0]
    b = packed.reshape(rows, k // group, nbytes).to(torch.int64)
    byte_shifts = torch.arange(nbytes, device=packed.device, dtype=torch.int64) * 8
    word = (b << byte_shifts).sum(dim=-1)
    shifts = torch.arange(group, device=packed.device, dtype=torch.int64) * bits
    return ((word.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)).reshape(rows, k)


def _nearest_code(x, elem):
    """Code of the nearest representable value; a tie goes to the even code.

    The non-negative codes of these formats ascend with their values, so the
    neighbours of |x| come from one sorted search; the sign bit is added back.
    """
    values = _values(elem, x.device)
    half = values.numel() // 2
    pos = values[:half]  # codes 0..half-1, ascending from 0
    mag = x.abs().clamp(max=float(pos[-1]))
    hi = torch.searchsorted(pos, mag.contiguous(), right=False).clamp(1, half - 1)
    lo = hi - 1
    dlo, dhi = mag - pos[lo], pos[hi] - mag
    take_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    code = torch.where(take_hi, hi, lo)
    negative = torch.signbit(x) & ~((code == 0) & (x == 0))
    # The reference's scan keeps +0 for zero-valued inputs and for negative
    # values that round to zero it lands on code 0 as well (the first of the
    # two equal-distance zeros it meets).
    negative = negative & (code != 0)
    return (code + negative.to(code.dtype) * half).to(torch.int32)


def pack(x, elem):
    """Pack `(rows, K)` values to dense `elem` codes along K.

    Args:
        x: values; K a multiple of 4 for the 6-bit elements, of 2 for e2m1.
        elem: "e3m2", "e2m3" or "e2m1".

    Returns:
        uint8 `(rows, K * bits / 8)`.
    """
    return _pack_bits(_nearest_code(x.float(), elem), SMALL_FLOATS[elem][2])


def unpack(packed, elem, k):
    """Unpack `elem` codes written by `pack` to `(rows, k)` float32 values."""
    bits = SMALL_FLOATS[elem][2]
    return _values(elem, packed.device)[_unpack_bits(packed.view(torch.uint8), k, bits)]


def round_tf32(x):
    """Round float32 to the 10 mantissa bits tf32 keeps (add half, clear 13 bits)."""
    return ((x.view(torch.int32) + 0x1000) & ~0x1FFF).view(torch.float32)


def to_blocked(scales):
    """`(rows, K / block)` scales -> the flat 128x4 blocked layout cuBLAS and
    torch._scaled_mm consume: 512-byte atoms ordered [row block][column group],
    the scale of row r, column c of an atom at byte (r % 32) * 16 + (r // 32) * 4 + c.
    Rows pad to 128 and columns to 4 with zeros."""
    rows, cols = scales.shape
    rb, cb = -(-rows // 128), -(-cols // 4)
    padded = torch.zeros((rb * 128, cb * 4), dtype=scales.dtype, device=scales.device)
    padded[:rows, :cols] = scales
    # [rb, 4 quarters, 32 rows, cb, 4 cols] -> [rb, cb, 32 rows, 4 quarters, 4 cols]
    atoms = padded.view(rb, 4, 32, cb, 4).permute(0, 3, 2, 1, 4)
    return atoms.reshape(-1).contiguous()


def _scale_buffers(d, rows, k, device, raw, blocked):
    block = sf_block(d)
    raw_t = torch.empty((rows, k // block), dtype=torch.uint8, device=device) if raw else None
    blocked_t = None
    if blocked:
        nbytes = (-(-rows // 128) * 128) * (-(-k // (block * 4)) * 4)
        blocked_t = torch.empty((nbytes,), dtype=torch.uint8, device=device)
    return raw_t, blocked_t


def _quantize_cuda(x, name, raw, blocked):
    """The CUDA path: one kernel writes the packed operand and the scales."""
    from . import capi

    d = DTYPES[name]
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.float()
    x = x.contiguous()
    rows, k = x.shape
    packed = torch.empty((rows, k * d.bits // 8), dtype=torch.uint8, device=x.device)
    raw_t, blocked_t = _scale_buffers(d, rows, k, x.device, raw, blocked)
    capi.library("smm").quantize(name, x, packed, raw_t, blocked_t)
    return (packed.view(d.a), None if raw_t is None else raw_t.view(d.sf),
            None if blocked_t is None else blocked_t.view(d.sf))


def quantize_blocked(x, name):
    """Quantise and lay the scales out for `gemm` in one step.

    Returns:
        `(packed, blocked_scales)`: what `gemm(a, b, sfa, sfb)` takes.  On a CUDA
        tensor this is a single kernel; on the CPU it is `quantize` + `to_blocked`.
    """
    if x.is_cuda:
        packed, _, blocked = _quantize_cuda(x, name, raw=False, blocked=True)
        return packed, blocked
    packed, scales = quantize(x, name)
    return packed, to_blocked(scales)


def quantize(x, name):
    """Quantise `(rows, K)` values to a block-scaled format.

    Args:
        x: values, K a multiple of the format's scale block.
        name: "nvfp4", "mxfp8" or "mxfp4".

    Returns:
        `(packed, scales)`: the operand in the format's torch dtype and the
        `(rows, K / block)` scales in the scale dtype, not yet blocked.  CUDA
        tensors go through the library's quantisation kernel, CPU tensors
        through the torch arithmetic below; both give the same bytes.
    """
    if x.is_cuda:
        packed, scales, _ = _quantize_cuda(x, name, raw=True, blocked=False)
        return packed, scales
    d = DTYPES[name]
    elem = elems(name)[0]
    block = sf_block(d)
    rows, k = x.shape
    groups = x.float().reshape(rows, k // block, block)
    top = 6.0 if d.bits == 4 else 448.0  # largest e2m1 / e4m3 magnitude
    scale = (groups.abs().amax(dim=-1, keepdim=True) / top).clamp(min=1e-30)
    if d.sf is torch.float8_e8m0fnu:
        scale = torch.pow(2.0, torch.ceil(torch.log2(scale)))  # power-of-two scales, rounded up
    stored = scale.squeeze(-1).to(d.sf)
    data = (groups / stored.float().unsqueeze(-1).clamp(min=1e-30)).reshape(rows, k).to(torch.bfloat16)
    if elem in SMALL_FLOATS:
        return pack(data, elem).view(d.a), stored
    return data.to(d.a), stored
