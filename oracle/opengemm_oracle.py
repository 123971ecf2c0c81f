"""CPU oracle for the OpenGEMM hot path: TEST INFRASTRUCTURE, not product code.

A numpy restatement of what aramesh10/OpenGEMM v0.1.4 computes for
`gemm(a, b[, sfa, sfb])`, C[M, N] = A[M, K] . B[N, K]^T, and of the packing,
quantising and scale-layout helpers either side of it.  Every function names
the reference file:line it follows.  Operands cross this module as raw bytes
(numpy uint8 / uint16 / float32 / int8 arrays), never as torch tensors, so the
same buffers can be handed to the C ABI of the CUDA library and to the oracle.

Only the test-suite, the smoke check and the `cpu_baseline` / `--impl
reference` legs of the benchmark may import this module; the product
(`opengemm_b200`) never does and fails loudly without its CUDA library.

Parity pin: the reference holds no golden vectors for this path
(its only check is kernel-vs-`bench.reference` on seeded inputs,
scripts/test.py:33-48).  The pin is therefore made against outputs of the
reference's own Python (quant.py, bench.py) imported on a CPU, stored under
tests/golden/ by tests/golden/make_golden.py, and checked by
tests/test_oracle_golden.py.
"""

from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------
# Format table.  opengemm/python/dtypes.py:37-53 (DTYPES) restated without
# torch: storage container, bits per value, output type, scale type.
# --------------------------------------------------------------------------

FORMATS = {
    #  name        impl   a-elem  b-elem  bits out     sf
    "bf16": ("mm", "bf16", "bf16", 16, "f32", None),
    "f16": ("mm", "f16", "f16", 16, "f32", None),
    "tf32": ("mm", "tf32", "tf32", 32, "f32", None),
    "s8": ("mm", "s8", "s8", 8, "s32", None),
    "u8": ("mm", "u8", "u8", 8, "s32", None),
    "e4m3": ("mm", "e4m3", "e4m3", 8, "f32", None),
    "e5m2": ("mm", "e5m2", "e5m2", 8, "f32", None),
    "e3m2": ("mm", "e3m2", "e3m2", 6, "f32", None),
    "e2m3": ("mm", "e2m3", "e2m3", 6, "f32", None),
    "e2m1": ("mm", "e2m1", "e2m1", 4, "f32", None),
    "e4m3xe5m2": ("mm", "e4m3", "e5m2", 8, "f32", None),
    "nvfp4": ("smm", "e2m1", "e2m1", 4, "bf16", "ue4m3"),
    "mxfp8": ("smm", "e4m3", "e4m3", 8, "bf16", "ue8m0"),
    "mxfp4": ("smm", "e2m1", "e2m1", 4, "bf16", "ue8m0"),
}

# opengemm/python/quant.py:8  (exponent bits, mantissa bits, storage bits)
SMALL_FLOATS = {"e3m2": (3, 2, 6), "e2m3": (2, 3, 6), "e2m1": (2, 1, 4)}


def impl_of(name):
    return FORMATS[name][0]


def bits_of(name):
    return FORMATS[name][3]


def sf_block(name):
    """Values per scale: 16 under ue4m3 scales, 32 under ue8m0 (dtypes.py:131-133)."""
    return 16 if FORMATS[name][5] == "ue4m3" else 32


def extent(name, k):
    """Bytes-or-elements row extent as the caller stores it (dtypes.py:123-125)."""
    bits = bits_of(name)
    return k * bits // 8 if bits < 8 else k


def scale_bytes(name, rows, k):
    """Bytes of a blocked scale tensor (api.py:20-22)."""
    return (-(-rows // 128) * 128) * (-(-k // (sf_block(name) * 4)) * 4)


# --------------------------------------------------------------------------
# Decoding the storage formats to float32.
# --------------------------------------------------------------------------


def small_float_values(elem):
    """Every code of a 4/6-bit float as its value, in code order (quant.py:10-24)."""
    exp_bits, mant_bits, _ = SMALL_FLOATS[elem]
    bias = (1 << (exp_bits - 1)) - 1
    out = []
    for code in range(1 << (1 + exp_bits + mant_bits)):
        sign = -1.0 if code >> (exp_bits + mant_bits) else 1.0
        exponent = (code >> mant_bits) & ((1 << exp_bits) - 1)
        mantissa = code & ((1 << mant_bits) - 1)
        if exponent == 0:
            mag = mantissa / (1 << mant_bits) * 2.0 ** (1 - bias)
        else:
            mag = (1 + mantissa / (1 << mant_bits)) * 2.0 ** (exponent - bias)
        out.append(sign * mag)
    return np.asarray(out, dtype=np.float32)


def _fp8_table(exp_bits, mant_bits, bias, fn):
    """All 256 codes of an 8-bit float.  `fn` = the e4m3fn flavour: no
    infinities, only S.1111.111 is NaN."""
    table = np.zeros(256, dtype=np.float32)
    emax = (1 << exp_bits) - 1
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exponent = (code >> mant_bits) & emax
        mantissa = code & ((1 << mant_bits) - 1)
        if fn:
            if exponent == emax and mantissa == (1 << mant_bits) - 1:
                table[code] = np.nan
                continue
        elif exponent == emax:
            table[code] = np.nan if mantissa else sign * np.inf
            continue
        if exponent == 0:
            mag = mantissa / (1 << mant_bits) * 2.0 ** (1 - bias)
        else:
            mag = (1 + mantissa / (1 << mant_bits)) * 2.0 ** (exponent - bias)
        table[code] = sign * mag
    return table


E4M3_TABLE = _fp8_table(4, 3, 7, fn=True)  # torch.float8_e4m3fn
E5M2_TABLE = _fp8_table(5, 2, 15, fn=False)  # torch.float8_e5m2


def _e8m0_table():
    """float8_e8m0fnu: 2^(code-127), code 255 is NaN."""
    with np.errstate(over="ignore"):
        table = np.ldexp(np.float32(1.0), np.arange(256, dtype=np.int32) - 127).astype(np.float32)
    table[255] = np.nan
    return table


E8M0_TABLE = _e8m0_table()


def bf16_to_f32(bits):
    """uint16 bfloat16 bit patterns -> float32 (the upcast of `t.float()`, bench.py:118-122)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x):
    """float32 -> bfloat16 bits, round to nearest even (`.to(torch.bfloat16)`, bench.py:137)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1)))) >> 16
    nan = np.isnan(x)
    out = rounded.astype(np.uint16)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def decode(elem, raw, k):
    """A `(rows, extent)` storage array as `(rows, k)` float32 values.

    Follows `_values` (bench.py:118-122): small floats through `unpack`,
    everything else `t.float()`.  Integers come back as float64 because the
    reference multiplies them as doubles (bench.py:139-140).
    """
    if elem in SMALL_FLOATS:
        return unpack(raw, elem, k)
    if elem == "bf16":
        return bf16_to_f32(raw)
    if elem == "f16":
        return np.asarray(raw).view(np.float16).astype(np.float32)
    if elem == "tf32":
        return np.asarray(raw, dtype=np.float32)
    if elem == "e4m3":
        return E4M3_TABLE[np.asarray(raw).view(np.uint8)]
    if elem == "e5m2":
        return E5M2_TABLE[np.asarray(raw).view(np.uint8)]
    if elem == "s8":
        return np.asarray(raw).view(np.int8).astype(np.float64)
    if elem == "u8":
        return np.asarray(raw).view(np.uint8).astype(np.float64)
    raise KeyError(elem)


def decode_scale(sf, raw):
    table = E4M3_TABLE if sf == "ue4m3" else E8M0_TABLE
    return table[np.asarray(raw).view(np.uint8)]


# --------------------------------------------------------------------------
# Bit packing of the 6- and 4-bit elements (quant.py:26-75).
# --------------------------------------------------------------------------


def pack_bits(codes, bits):
    """Dense little-end-first packing: value 0 in the low bits; four 6-bit
    codes to three bytes, two 4-bit codes to one (quant.py:26-35)."""
    per_word = {6: 4, 4: 2}[bits]
    out_bytes = per_word * bits // 8
    rows, k = codes.shape
    q = codes.reshape(rows, k // per_word, per_word).astype(np.int64)
    word = np.zeros(q.shape[:2], dtype=np.int64)
    for i in range(per_word):
        word |= q[..., i] << (bits * i)
    packed = np.stack([(word >> (8 * b)) & 0xFF for b in range(out_bytes)], axis=-1)
    return packed.reshape(rows, k // per_word * out_bytes).astype(np.uint8)


def unpack_bits(packed, k, bits):
    """Inverse of `pack_bits` (quant.py:37-48)."""
    per_word = {6: 4, 4: 2}[bits]
    out_bytes = per_word * bits // 8
    packed = np.asarray(packed).view(np.uint8)
    rows = packed.shape[0]
    b = packed.reshape(rows, k // per_word, out_bytes).astype(np.int64)
    word = np.zeros(b.shape[:2], dtype=np.int64)
    for i in range(out_bytes):
        word |= b[..., i] << (8 * i)
    mask = (1 << bits) - 1
    return np.stack([(word >> (bits * i)) & mask for i in range(per_word)], axis=-1).reshape(rows, k)


def nearest_code(x, elem):
    """The code of the representable value nearest each x; a tie goes to the
    even code.  The reference scans codes in order and replaces the running
    best on a strictly smaller distance, or on an equal distance when the
    candidate is even and the holder odd (quant.py:58-69); the scan below is
    that loop."""
    values = small_float_values(elem)
    x = np.asarray(x, dtype=np.float32)
    code = np.zeros(x.shape, dtype=np.int32)
    best = np.abs(x - values[0])
    for c in range(1, values.size):
        distance = np.abs(x - values[c])
        take = (distance < best) | ((distance == best) & (c % 2 == 0) & (code % 2 == 1))
        best = np.where(take, distance, best)
        code = np.where(take, c, code)
    return code


def pack(x, elem):
    """Values -> dense `elem` codes along K (quant.py:50-70)."""
    return pack_bits(nearest_code(x, elem), SMALL_FLOATS[elem][2])


def unpack(packed, elem, k):
    """Dense `elem` codes -> float32 values (quant.py:72-75)."""
    return small_float_values(elem)[unpack_bits(packed, k, SMALL_FLOATS[elem][2])]


def round_tf32(x):
    """float32 rounded to tf32's 10 mantissa bits: add half, clear 13 bits (quant.py:77-80)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.int32)
    return ((bits + np.int32(0x1000)) & np.int32(~0x1FFF)).view(np.float32)


# --------------------------------------------------------------------------
# The 128x4 blocked scale layout (quant.py:82-97).
# --------------------------------------------------------------------------


def to_blocked(scales):
    """`(rows, cols)` one-byte scales -> flat blocked buffer.

    Rows pad to 128 and columns to 4 with zero bytes.  The buffer is a
    sequence of 512-byte atoms ordered [row block][column group]; inside an
    atom the scale of row r, column c sits at byte (r%32)*16 + (r//32)*4 + c.
    """
    scales = np.asarray(scales).view(np.uint8)
    rows, cols = scales.shape
    rb, cb = -(-rows // 128), -(-cols // 4)
    padded = np.zeros((rb * 128, cb * 4), dtype=np.uint8)
    padded[:rows, :cols] = scales
    atoms = padded.reshape(rb, 128, cb, 4).transpose(0, 2, 1, 3)  # rb, cb, 128, 4
    return np.ascontiguousarray(atoms.reshape(-1, 4, 32, 4).transpose(0, 2, 1, 3)).reshape(-1)


def from_blocked(flat, rows, cols):
    """Inverse of `to_blocked`: the `(rows, cols)` scales a blocked buffer holds."""
    rb, cb = -(-rows // 128), -(-cols // 4)
    flat = np.asarray(flat).view(np.uint8)[: rb * cb * 512]
    atoms = flat.reshape(rb * cb, 32, 4, 4).transpose(0, 2, 1, 3).reshape(rb, cb, 128, 4)
    return np.ascontiguousarray(atoms.transpose(0, 2, 1, 3)).reshape(rb * 128, cb * 4)[:rows, :cols]


# --------------------------------------------------------------------------
# float32 -> one-byte float conversions that torch's `.to(dtype)` performs in
# the reference's quantize (quant.py:115-121).
# --------------------------------------------------------------------------


def _nearest_even_from_table(x, table_pos):
    """Round non-negative x to the nearest entry of an ascending table, a tie
    going to the even index."""
    idx = np.searchsorted(table_pos, x, side="left")
    idx = np.clip(idx, 1, table_pos.size - 1)
    lo, hi = table_pos[idx - 1], table_pos[idx]
    dlo, dhi = x - lo, hi - x
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (idx % 2 == 0))
    return np.where(pick_hi, idx, idx - 1)


def f32_to_e4m3(x):
    """float32 -> float8_e4m3fn codes: nearest even; magnitudes that round
    past 448 (>= 464 after the tie rule, i.e. > 464 or the 480 boundary)
    become NaN as torch's cast does."""
    x = np.asarray(x, dtype=np.float32)
    pos = np.append(E4M3_TABLE[:0x7F].astype(np.float64), 480.0)  # codes 0..0x7E, then the NaN slot
    mag = np.abs(x).astype(np.float64)
    idx = _nearest_even_from_table(np.minimum(mag, 1e9), pos)
    idx = np.where(np.isnan(x), 0x7F, idx)
    return (idx | np.where(np.signbit(x), 0x80, 0)).astype(np.uint8)


def f32_to_e5m2(x):
    """float32 -> float8_e5m2 codes, nearest even, overflow to infinity."""
    x = np.asarray(x, dtype=np.float32)
    finite = E5M2_TABLE[:0x7C].astype(np.float64)
    pos = np.append(finite, 65536.0)  # index 0x7C = inf
    mag = np.abs(x).astype(np.float64)
    idx = _nearest_even_from_table(np.minimum(mag, 1e9), pos)
    idx = np.where(np.isnan(x), 0x7F, idx)
    return (idx | np.where(np.signbit(x), 0x80, 0)).astype(np.uint8)


def pow2_to_e8m0(x):
    """Exact powers of two -> float8_e8m0fnu codes (biased exponent 127)."""
    _, e = np.frexp(np.asarray(x, dtype=np.float32))  # x = 0.5 * 2^e
    return np.clip(e - 1 + 127, 0, 254).astype(np.uint8)


def quantize(x, name):
    """`(rows, K)` values -> `(packed storage, (rows, K/block) scale bytes)`.

    Follows quant.py:99-122 step for step: per block scale = amax / 6 (4-bit)
    or / 448 (e4m3) floored at 1e-30; for ue8m0 scales rounded UP to a power of
    two; the stored scale is that value cast to the scale type; the data is
    value / float(stored scale), rounded through bfloat16, then to the
    nearest element value.
    """
    impl, elem, _, bits, _, sf = FORMATS[name]
    assert impl == "smm"
    block = sf_block(name)
    x = np.asarray(x, dtype=np.float32)
    rows, k = x.shape
    blocks = x.reshape(rows, k // block, block)
    amax = np.float32(6.0 if bits == 4 else 448.0)
    scale = np.maximum(np.abs(blocks).max(axis=-1, keepdims=True) / amax, np.float32(1e-30))
    if sf == "ue8m0":
        scale = np.exp2(np.ceil(np.log2(scale))).astype(np.float32)
        stored = pow2_to_e8m0(scale[..., 0])
    else:
        stored = f32_to_e4m3(scale[..., 0])
    stored_f = np.maximum(decode_scale(sf, stored), np.float32(1e-30))[..., None]
    data = (blocks / stored_f).astype(np.float32).reshape(rows, k)
    data = bf16_to_f32(f32_to_bf16(data))
    if elem in SMALL_FLOATS:
        return pack(data, elem), stored
    return f32_to_e4m3(data), stored


# --------------------------------------------------------------------------
# The reference product (bench.py:125-144) and its acceptance rule.
# --------------------------------------------------------------------------


def dequantize(name, raw, sf_raw, k, which="a"):
    """Storage (+ unblocked scale bytes) -> the float operand the product is taken of."""
    _, ea, eb, _, _, sf = FORMATS[name]
    values = decode(ea if which == "a" else eb, raw, k)
    if sf is None:
        return values
    scale = decode_scale(sf, sf_raw)
    return values * np.repeat(scale, sf_block(name), axis=1)[:, :k]


def reference(name, a, b, sfa_raw=None, sfb_raw=None):
    """C = A . B^T as the reference's oracle defines it (bench.py:125-144).

    float formats: float32 matmul of the upcast operands -> float32;
    s8/u8: float64 matmul (exact) -> int32;
    block-scaled: float32 matmul of values x repeated scales -> bfloat16 bits
    (returned as uint16).
    """
    impl, _, _, bits, out, _ = FORMATS[name]
    a = np.asarray(a)
    k = a.shape[1] * 8 // bits if bits < 8 else a.shape[1]
    fa = dequantize(name, a, sfa_raw, k, "a")
    fb = dequantize(name, b, sfb_raw, k, "b")
    if out == "s32":
        return np.rint(fa @ fb.T).astype(np.int32)
    c = fa.astype(np.float32) @ fb.astype(np.float32).T
    if out == "bf16":
        return f32_to_bf16(c)
    return c


# (rtol, atol) at K = 4096 (bench.py:28-35); both grow with sqrt(K/4096) (bench.py:71-75).
TOLERANCE = {
    "s8": (0.0, 0.0),
    "u8": (0.0, 0.0),
    "nvfp4": (2.0**-6, 2.0**-5),
    "mxfp8": (2.0**-6, 2.0**-5),
    "mxfp4": (2.0**-6, 2.0**-5),
}
DEFAULT_TOLERANCE = (1.0e-3, 2.0e-2)


def tolerance(name, k):
    rtol, atol = TOLERANCE.get(name, DEFAULT_TOLERANCE)
    scale = max(1.0, (k / 4096) ** 0.5)
    return rtol * scale, atol * scale


def as_float(name, c):
    """An output buffer (float32 / int32 / bf16 bits) as float64 for comparison."""
    out = FORMATS[name][4]
    if out == "bf16":
        return bf16_to_f32(np.asarray(c).view(np.uint16)).astype(np.float64)
    return np.asarray(c).astype(np.float64)


def check_close(name, k, got, want):
    """The reference's acceptance rule, `assert_close(got, want, rtol, atol)`
    (scripts/test.py:47-48): |got - want| <= atol + rtol * |want| everywhere.
    Returns (ok, worst excess)."""
    rtol, atol = tolerance(name, k)
    g, w = as_float(name, got), as_float(name, want)
    excess = np.abs(g - w) - (atol + rtol * np.abs(w))
    bad = ~(excess <= 0)  # NaN counts as a failure
    return (not bad.any()), float(np.nanmax(excess)) if excess.size else 0.0


def bf16_ulp(x):
    """One bfloat16 unit in the last place at |x| (float64 in, float64 out)."""
    x = np.abs(np.asarray(x, dtype=np.float64))
    e = np.floor(np.log2(np.maximum(x, 2.0**-126)))
    return 2.0 ** (e - 7)


def check_north_star(name, got, want):
    """The stricter acceptance stated for this build.

    s8/u8: bit-exact.  Dense float formats with f32 output: max|got-want| /
    max|want| <= 1e-3.  Block-scaled bf16 output: |got-want| <= 1 bf16 ulp of
    want + 1e-2 * |want|, plus 2^-20 of the largest |want| as the floor a
    float32 sum of cancelling terms cannot go below (outputs that cancel to
    nearly zero have an ulp far smaller than either side's rounding of the
    sum).  Returns (ok, figure of merit)."""
    out = FORMATS[name][4]
    g, w = as_float(name, got), as_float(name, want)
    if out == "s32":
        diff = np.abs(g - w).max() if g.size else 0.0
        return bool(diff == 0), float(diff)
    if out == "f32":
        denom = max(float(np.abs(w).max()), 1e-30) if w.size else 1.0
        err = float(np.abs(g - w).max() / denom) if g.size else 0.0
        return bool(err <= 1e-3), err
    floor = 2.0**-20 * (float(np.abs(w).max()) if w.size else 0.0)
    excess = np.abs(g - w) - (bf16_ulp(w) + 1e-2 * np.abs(w) + floor)
    ok = bool((excess <= 0).all())
    return ok, float(excess.max()) if excess.size else 0.0


def north_star_floor_users(name, got, want):
    """How many block-scaled outputs pass `check_north_star` only because of
    its 2^-20 * max|want| floor: outputs within (1 bf16 ulp + 1e-2 |want| +
    floor) but outside (1 bf16 ulp + 1e-2 |want|).  Reported beside parity
    results so the floor's reach is visible; 0 for the other output types."""
    if FORMATS[name][4] != "bf16":
        return 0
    g, w = as_float(name, got), as_float(name, want)
    bare = np.abs(g - w) - (bf16_ulp(w) + 1e-2 * np.abs(w))
    floor = 2.0**-20 * (float(np.abs(w).max()) if w.size else 0.0)
    return int(((bare > 0) & (bare <= floor)).sum())


def check_bf16_output(got_bits, want_f32):
    """Acceptance for a dense format whose f32 accumulator is rounded to
    bfloat16 on the way out (an output variant this build adds; the reference
    has none, so the rule is stated here): every output within one bfloat16
    unit in the last place of the float32 reference, plus 2^-20 of the largest
    |reference| (sums that cancel to nearly zero carry the rounding of their
    terms, not of their value).  Returns (ok, worst excess in ulps)."""
    got = bf16_to_f32(np.asarray(got_bits).view(np.uint16)).astype(np.float64)
    want = np.asarray(want_f32, dtype=np.float64)
    floor = 2.0**-20 * (float(np.abs(want).max()) if want.size else 0.0)
    ulp = bf16_ulp(want)
    excess = (np.abs(got - want) - floor) / ulp
    bad = ~(excess <= 1.0)
    return (not bad.any()), float(np.nanmax(excess)) if excess.size else 0.0


def f16_ulp(x):
    """One IEEE half unit in the last place at |x| (subnormals below 2^-14 share 2^-24)."""
    x = np.abs(np.asarray(x, dtype=np.float64))
    e = np.floor(np.log2(np.maximum(x, 2.0**-14)))
    return 2.0 ** (e - 10)


def check_f16_output(got_bits, want_f32):
    """Acceptance for a dense format whose f32 accumulator is rounded to IEEE
    half on the way out (an output variant this build adds): every output
    within one half unit in the last place of the float32 reference, plus
    2^-16 of the largest |reference|.  The floor is the accumulation's own
    error - the tensor cores' sums of K products differ from a float32 matmul
    by a few 2^-20 of the largest output (more for tf32 operands), which a
    half's 11-bit significand resolves where bfloat16's 8 bits do not; it
    stays 64 times tighter than the 1e-3 bound on float32 output.
    Returns (ok, worst excess in ulps)."""
    got = np.asarray(got_bits).view(np.float16).astype(np.float64)
    want = np.asarray(want_f32, dtype=np.float64)
    floor = 2.0**-16 * (float(np.abs(want).max()) if want.size else 0.0)
    excess = (np.abs(got - want) - floor) / f16_ulp(want)
    bad = ~(excess <= 1.0)
    return (not bad.any()), float(np.nanmax(excess)) if excess.size else 0.0
