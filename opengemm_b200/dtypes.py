"""The fourteen operand formats, as the torch front end sees them.

Same public names and meaning as the reference's table and helpers
(opengemm/python/dtypes.py:28-133): `DTYPES[name]` has fields
`impl, a, b, bits, out, sf`; `dtype_name` resolves operands or element names
to a key; `extent` / `k_of` convert between K in values and the row extent
torch sees; `sf_block` is the number of values one scale covers.
"""

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Dtype:
    impl: str  # "mm": dense, "smm": block-scaled
    a: torch.dtype
    b: torch.dtype
    bits: int  # per value; below 8 the values are packed along K
    out: torch.dtype
    sf: object  # torch dtype of the scales, None for dense formats
    elem_a: str = ""
    elem_b: str = ""

    def __iter__(self):  # unpacks like the reference's NamedTuple
        return iter((self.impl, self.a, self.b, self.bits, self.out, self.sf))


_T = torch
_FP4X2 = torch.float4_e2m1fn_x2
_ROWS = [
    # name, impl, torch a, torch b, bits, out, scales, element a, element b
    ("bf16", "mm", _T.bfloat16, _T.bfloat16, 16, _T.float32, None, "bf16", "bf16"),
    ("f16", "mm", _T.float16, _T.float16, 16, _T.float32, None, "f16", "f16"),
    ("tf32", "mm", _T.float32, _T.float32, 32, _T.float32, None, "tf32", "tf32"),
    ("s8", "mm", _T.int8, _T.int8, 8, _T.int32, None, "s8", "s8"),
    ("u8", "mm", _T.uint8, _T.uint8, 8, _T.int32, None, "u8", "u8"),
    ("e4m3", "mm", _T.float8_e4m3fn, _T.float8_e4m3fn, 8, _T.float32, None, "e4m3", "e4m3"),
    ("e5m2", "mm", _T.float8_e5m2, _T.float8_e5m2, 8, _T.float32, None, "e5m2", "e5m2"),
    ("e3m2", "mm", _T.uint8, _T.uint8, 6, _T.float32, None, "e3m2", "e3m2"),
    ("e2m3", "mm", _T.uint8, _T.uint8, 6, _T.float32, None, "e2m3", "e2m3"),
    ("e2m1", "mm", _T.uint8, _T.uint8, 4, _T.float32, None, "e2m1", "e2m1"),
    ("e4m3xe5m2", "mm", _T.float8_e4m3fn, _T.float8_e5m2, 8, _T.float32, None, "e4m3", "e5m2"),
    ("nvfp4", "smm", _FP4X2, _FP4X2, 4, _T.bfloat16, _T.float8_e4m3fn, "e2m1", "ue4m3"),
    ("mxfp8", "smm", _T.float8_e4m3fn, _T.float8_e4m3fn, 8, _T.bfloat16, _T.float8_e8m0fnu, "e4m3", "ue8m0"),
    ("mxfp4", "smm", _FP4X2, _FP4X2, 4, _T.bfloat16, _T.float8_e8m0fnu, "e2m1", "ue8m0"),
]
DTYPES = {row[0]: Dtype(*row[1:]) for row in _ROWS}

# An addition with no counterpart in the reference: every dense float format
# can round its f32 accumulator to bfloat16 or to IEEE half on the way out,
# which halves the bytes of C.  The native library knows these as
# "<format>.bf16" / "<format>.f16"; `DTYPES` itself stays the reference's
# fourteen.
BF16_OUT_SUFFIX = ".bf16"
NARROW_OUT_SUFFIXES = {torch.bfloat16: ".bf16", torch.float16: ".f16"}
NARROW_OUT = {
    row[0] + suffix: Dtype(row[1], row[2], row[3], row[4], out, row[6], row[7], row[8])
    for row in _ROWS
    if row[1] == "mm" and row[5] is torch.float32
    for out, suffix in NARROW_OUT_SUFFIXES.items()
}
BF16_OUT = {name: d for name, d in NARROW_OUT.items() if name.endswith(BF16_OUT_SUFFIX)}


def lookup(name):
    """The `Dtype` of one of the fourteen formats or of a 2-byte-output variant."""
    found = DTYPES.get(name) or NARROW_OUT.get(name)
    if found is None:
        raise TypeError(f"{name} is not a format this build serves; have {list(DTYPES)} "
                        f"(+ {' / '.join(map(repr, NARROW_OUT_SUFFIXES.values()))} on dense float formats)")
    return found


def base_name(name):
    """The reference format a name belongs to ("e4m3.bf16" -> "e4m3")."""
    for suffix in NARROW_OUT_SUFFIXES.values():
        if name.endswith(suffix):
            return name[: -len(suffix)]
    return name

# Dense formats torch can name by dtype alone: both operands alike and not
# uint8, which carries four different elements.
_DENSE_BY_TORCH = {
    d.a: name for name, d in DTYPES.items() if d.impl == "mm" and d.a is d.b and d.a is not torch.uint8
}
_SCALED_BY_TORCH = {(d.a, d.sf): name for name, d in DTYPES.items() if d.impl == "smm"}


def elems(name):
    """Element names of a format: `(a, b)` when dense, `(element, scale)` when block-scaled."""
    d = DTYPES[name]
    return d.elem_a, d.elem_b


def _element_of(t, which):
    name = _DENSE_BY_TORCH.get(t.dtype)
    if name is None:
        raise TypeError(
            f"{which} is {t.dtype}, which names no element: pass {which}type= "
            f"(uint8 carries u8, e3m2, e2m3 and e2m1 alike; the rest are inferred)"
        )
    return name


def dtype_name(a=None, b=None, sfa=None, atype=None, btype=None, sftype=None):
    """The `DTYPES` key for these operands, or for these element names.

    With scales the key follows from the operand and scale dtypes.  Without,
    each operand's element is its `atype=` / `btype=` name or is inferred from
    its torch dtype (uint8 must be named); two different elements join as
    "axb".  With no operands at all, `atype` (and `sftype` "ue4m3" / "ue8m0"
    for a block-scaled format) name the format.

    Raises:
        TypeError: when nothing served matches.
    """
    if sfa is not None:
        key = (a.dtype, sfa.dtype)
        if key not in _SCALED_BY_TORCH:
            raise TypeError(
                f"{a.dtype} operands with {sfa.dtype} scales is not a format; have {_SCALED_BY_TORCH}"
            )
        return _SCALED_BY_TORCH[key]
    if sftype is not None:
        for name, d in DTYPES.items():
            if d.impl == "smm" and elems(name) == (atype, sftype):
                return name
        raise TypeError(f"atype={atype!r} with sftype={sftype!r} is not a format")
    if a is not None:
        atype = atype or _element_of(a, "a")
        if not btype:
            btype = atype if b.dtype == a.dtype else _element_of(b, "b")
    if atype is None:
        raise TypeError("without operands, pass atype= (and sftype= for a block-scaled format)")
    name = atype if btype in (None, atype) else f"{atype}x{btype}"
    if name not in DTYPES:
        raise TypeError(f"{name} is not a format this build serves; have {list(DTYPES)}")
    return name


def extent(d, k):
    """Row extent of a `(rows, K)` operand as torch sees it: packed bytes below 8 bits."""
    return k * d.bits // 8 if d.bits < 8 else k


def k_of(d, row_extent):
    """K in values for a row extent; inverse of `extent`."""
    return row_extent * 8 // d.bits if d.bits < 8 else row_extent


def sf_block(d):
    """Values per scale: 16 with ue4m3 scales, 32 with ue8m0."""
    return 16 if d.sf is torch.float8_e4m3fn else 32
