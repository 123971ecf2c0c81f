"""ctypes binding of libopengemm_b200.so: the C ABI of include/opengemm_b200.h.

Mirrors the reference's binding layer (opengemm/python/capi.py:12-188): the
`OgGemm` structure, which config keys pick a kernel and which steer a launch,
`Library(impl)` with `kernels / bind / launch / error`, and the module-level
`library()` / `bind()`.  One shared object serves both `impl`s here.  There is
no fallback: a missing or unloadable library raises.
"""

import ctypes
import threading
from ctypes import POINTER, byref, c_char, c_char_p, c_int32, c_void_p

import torch

from . import build
from .dtypes import lookup

ABI_VERSION = 3
OG_OK, OG_ERR_BIND, OG_ERR_NO_KERNEL, OG_ERR_TENSORMAP, OG_ERR_LAUNCH, OG_ERR_TIMEOUT = 0, -1, -2, -3, -4, -5

_INT_FIELDS_BEFORE = ("m", "n", "k")
_INT_FIELDS_AFTER = (
    "use_2cta", "output_n", "use_clc", "swap_ab",
    "cluster_m", "cluster_n", "cluster_k",
    "block_m", "stages", "epi_hold", "epi_double", "epi_direct",
    "epi_trade", "deep_stages",
    "supergroup", "split_k", "walk", "l2_promo",
    "persistent",
    "row",
)


class OgGemm(ctypes.Structure):
    """One GEMM as the C side sees it (include/opengemm_b200.h, 108 bytes)."""

    _fields_ = (
        [(f, c_int32) for f in _INT_FIELDS_BEFORE]
        + [("dtype", c_char * 16)]
        + [(f, c_int32) for f in _INT_FIELDS_AFTER]
    )


assert ctypes.sizeof(OgGemm) == 108


class OgPlan(ctypes.Structure):
    """The native tile plan of a bound GEMM (og_b200_plan)."""

    _fields_ = [
        (f, c_int32)
        for f in (
            "cta_group", "tile_m", "tile_n", "block_k", "stages", "swap", "epi_staged", "epi_tma",
            "acc_slots", "tmem_cols", "smem_bytes", "tiles", "grid", "group", "stream_k", "use_clc", "fixed_shape", "cluster_k", "plain",
        )
    ]


# Config keys that pick a kernel, and those read at launch, per implementation
# (the split the reference makes in capi.py:36-67).
KERNEL_KEYS = {
    "mm": ("use_2cta", "output_n", "use_clc", "swap_ab", "cluster_m", "cluster_n", "cluster_k",
           "block_m", "stages", "epi_hold", "epi_double", "epi_direct", "split_k"),
    "smm": ("use_2cta", "output_n", "use_clc", "swap_ab", "cluster_m", "cluster_n", "cluster_k",
            "epi_trade", "deep_stages"),
}
LAUNCH_KEYS = {
    "mm": ("supergroup", "walk", "l2_promo"),
    # split_k, walk, stages and l2_promo are additions of this build for the block-scaled formats
    # (the struct has the fields; the reference's block-scaled library does not read them)
    "smm": ("supergroup", "epi_direct", "persistent", "split_k", "walk", "stages", "l2_promo"),
}
# Defaults for keys an entry may omit (entries written by this build's tuner carry all of them).
KEY_DEFAULTS = {
    "use_2cta": 0, "output_n": 128, "use_clc": 0, "swap_ab": 0, "cluster_m": 1, "cluster_n": 1,
    "cluster_k": 1, "block_m": 128, "stages": 0, "epi_hold": 1, "epi_double": 0, "epi_direct": 0,
    "split_k": 1, "epi_trade": 0, "deep_stages": 0, "supergroup": 8, "walk": 0, "l2_promo": 0,
    "persistent": 1,
}


def raw_stream(device):
    """The current CUDA stream of device index `device` as a raw handle."""
    try:
        return torch._C._cuda_getCurrentRawStream(device)
    except AttributeError:
        return torch.cuda.current_stream(device).cuda_stream


def scale_bytes(d, rows, k):
    """Bytes of a scale tensor in the 128x4 blocked layout."""
    from .dtypes import sf_block

    return (-(-rows // 128) * 128) * (-(-k // (sf_block(d) * 4)) * 4)


class Library:
    """The shared library seen through one implementation's six entry points."""

    def __init__(self, impl, path=None):
        """`path` loads another shared library that exports the same entry
        points (a measuring tool's use); by default the in-tree build."""
        self.impl = impl
        self.path = path if path is not None else build.library_path(impl)
        try:
            lib = ctypes.CDLL(str(self.path))
        except OSError as exc:
            raise RuntimeError(
                f"cannot load the {impl} kernel library {self.path}: {exc}; there is no CPU fallback"
            ) from exc
        self._lib = lib
        prefix = f"og_{impl}_"
        sig = {
            "abi": (c_int32, []),
            "error": (c_char_p, []),
            "kernels": (c_int32, []),
            "kernel": (c_int32, [c_int32, POINTER(OgGemm)]),
            "bind": (c_int32, [POINTER(OgGemm)]),
            "launch": (c_int32, [POINTER(OgGemm)] + [c_void_p] * 5 + [c_int32, c_void_p]),
        }
        for name, (restype, argtypes) in sig.items():
            fn = getattr(lib, prefix + name)
            fn.restype, fn.argtypes = restype, argtypes
            setattr(self, "_" + name, fn)
        found = self._abi()
        if found != ABI_VERSION:
            raise RuntimeError(
                f"{impl} library {self.path} is ABI version {found}, this build speaks {ABI_VERSION}; "
                f"delete it and let it rebuild"
            )
        # Additions of this build; absent when OPENGEMM_LIB_* points at another library.
        self._plan = getattr(lib, "og_b200_plan", None)
        if self._plan is not None:
            self._plan.restype, self._plan.argtypes = c_int32, [POINTER(OgGemm), c_int32, POINTER(OgPlan)]
            self._alpha = lib.og_b200_launch_alpha
            self._alpha.restype = c_int32
            self._alpha.argtypes = [POINTER(OgGemm)] + [c_void_p] * 5 + [c_int32, c_void_p, ctypes.c_float]
            self._checked = lib.og_b200_launch_checked
            self._checked.restype = c_int32
            self._checked.argtypes = [POINTER(OgGemm)] + [c_void_p] * 5 + [c_int32, c_void_p, c_void_p]
            self._set_limit = lib.og_b200_set_wait_limit_ms
            self._set_limit.restype, self._set_limit.argtypes = None, [c_int32]
            self._independent = lib.og_b200_set_independent_inputs
            self._independent.restype, self._independent.argtypes = None, [c_int32]
            self._quantize = lib.og_b200_quantize
            self._quantize.restype = c_int32
            self._quantize.argtypes = [c_char_p, c_void_p, c_int32, ctypes.c_int64, ctypes.c_int64, c_void_p, c_void_p,
                                       c_void_p, c_int32, c_void_p]
            self._quantize_error = lib.og_b200_quantize_error
            self._quantize_error.restype = c_char_p
            self._describe = lib.og_b200_describe
            self._describe.restype = c_int32
            self._describe.argtypes = [POINTER(OgGemm), c_int32, c_char_p, c_int32]
            self._bias = lib.og_b200_launch_bias
            self._bias.restype = c_int32
            self._bias.argtypes = [POINTER(OgGemm)] + [c_void_p] * 5 + [c_int32, c_void_p, ctypes.c_float, c_void_p]
            self._status = lib.og_b200_status
            self._status.restype, self._status.argtypes = c_int32, [c_int32]
            self._prepare = lib.og_b200_prepare_device
            self._prepare.restype, self._prepare.argtypes = c_int32, [c_int32]
            self._tile_order = lib.og_b200_tile_order
            self._tile_order.restype, self._tile_order.argtypes = c_int32, [POINTER(OgGemm), POINTER(c_int32), c_int32]
            self._overcredit = lib.og_b200_test_overcredit_next_launch
            self._overcredit.restype, self._overcredit.argtypes = None, [c_int32]
            self._quantized = lib.og_b200_launch_quantized
            self._quantized.restype = c_int32
            self._quantized.argtypes = [POINTER(OgGemm)] + [c_void_p] * 6 + [c_int32, c_void_p, c_char_p]
            self._fixed = lib.og_b200_set_fixed_kernels
            self._fixed.restype, self._fixed.argtypes = None, [c_int32]
        self._kernels = None

    def error(self):
        return self._error().decode()

    def kernels(self):
        """Every configuration this library offers, as configs.json dicts with a `dtype` key."""
        if self._kernels is None:
            rows = []
            for i in range(self._kernels_count()):
                g = OgGemm()
                self._kernel(i, byref(g))
                row = {"dtype": g.dtype.decode()}
                row.update({key: getattr(g, key) for key in KERNEL_KEYS[self.impl]})
                rows.append(row)
            self._kernels = rows
        return self._kernels

    def _kernels_count(self):
        return self._lib[f"og_{self.impl}_kernels"]()

    def spell(self, row):
        return " ".join(f"{key}={int(row[key])}" for key in KERNEL_KEYS[self.impl])

    def bind(self, name, m, n, k, config):
        """Resolve a configs.json entry for a shape.  Returns the OgGemm to launch
        with; it must not be edited afterwards."""
        keys = KERNEL_KEYS[self.impl] + LAUNCH_KEYS[self.impl]
        knobs = {key: int(config.get(key, KEY_DEFAULTS[key])) for key in keys}
        g = OgGemm(m=m, n=n, k=k, dtype=name.encode(), **knobs)
        status = self._bind(byref(g))
        if status == OG_OK:
            return g
        message = self.error()
        if status == OG_ERR_NO_KERNEL:
            message += f"\n\nrequested: {self.spell({k_: knobs.get(k_, 0) for k_ in KERNEL_KEYS[self.impl]})}"
        raise RuntimeError(message)

    def launch(self, g, a, b, sfa, sfb, out):
        """Enqueue the bound kernel on the current stream of the operands' device."""
        device = a.get_device()
        status = self._launch(
            byref(g), a.data_ptr(), b.data_ptr(),
            0 if sfa is None else sfa.data_ptr(), 0 if sfb is None else sfb.data_ptr(),
            out.data_ptr(), device, raw_stream(device),
        )
        if status != OG_OK:
            raise RuntimeError(self.error())

    def launcher(self, g, a, b, sfa, sfb, out):
        """A zero-argument callable that enqueues this launch on the current
        stream of the operands' device each time it is called.  The bound GEMM
        and the tensors' addresses are captured once (and the tensors kept
        alive), which leaves about a third of `launch`'s interpreter time per
        call: for loops that run the same buffers again and again, where a
        small GEMM is otherwise timed by the wrapper around it."""
        device = a.get_device()
        args = (byref(g), a.data_ptr(), b.data_ptr(), 0 if sfa is None else sfa.data_ptr(),
                0 if sfb is None else sfb.data_ptr(), out.data_ptr(), device)
        launch = self._launch

        def call():
            if launch(*args, raw_stream(device)) != OG_OK:
                raise RuntimeError(self.error())

        call.keeps = (g, a, b, sfa, sfb, out)  # the addresses above stay valid as long as the callable lives
        return call

    def launch_checked(self, g, a, b, sfa, sfb, out, status_word):
        """Like `launch`, with a zeroed int32 device tensor that receives a code
        if any device-side wait gives up."""
        device = a.get_device()
        status = self._checked(
            byref(g), a.data_ptr(), b.data_ptr(),
            0 if sfa is None else sfa.data_ptr(), 0 if sfb is None else sfb.data_ptr(),
            out.data_ptr(), device, raw_stream(device), status_word.data_ptr(),
        )
        if status != OG_OK:
            raise RuntimeError(self.error())

    def launch_alpha(self, g, a, b, sfa, sfb, out, alpha):
        """Like `launch`, every output multiplied by `alpha` in float32 before it is stored."""
        device = a.get_device()
        status = self._alpha(
            byref(g), a.data_ptr(), b.data_ptr(),
            0 if sfa is None else sfa.data_ptr(), 0 if sfb is None else sfb.data_ptr(),
            out.data_ptr(), device, raw_stream(device), float(alpha),
        )
        if status != OG_OK:
            raise RuntimeError(self.error())

    def launch_bias(self, g, a, b, sfa, sfb, out, alpha, bias):
        """Like `launch`, every output multiplied by `alpha` and the float32 vector `bias`
        (one value per column of C) added, in float32, before it is stored."""
        device = a.get_device()
        status = self._bias(
            byref(g), a.data_ptr(), b.data_ptr(),
            0 if sfa is None else sfa.data_ptr(), 0 if sfb is None else sfb.data_ptr(),
            out.data_ptr(), device, raw_stream(device), float(alpha), bias.data_ptr(),
        )
        if status != OG_OK:
            raise RuntimeError(self.error())

    def launch_quantized(self, g, a, b, sfa, sfb, packed, scales, out_format):
        """Like `launch`, with C leaving block-scaled: packed codes into `packed`,
        128x4 blocked scales into `scales`."""
        device = a.get_device()
        status = self._quantized(
            byref(g), a.data_ptr(), b.data_ptr(),
            0 if sfa is None else sfa.data_ptr(), 0 if sfb is None else sfb.data_ptr(),
            packed.data_ptr(), scales.data_ptr(), device, raw_stream(device), out_format.encode(),
        )
        if status != OG_OK:
            raise RuntimeError(self.error())

    def status(self, word):
        """OG_OK for a zero status word of `launch_checked`, else OG_ERR_TIMEOUT with
        `error()` naming the wait that gave up."""
        return self._status(int(word))

    def prepare_device(self, device):
        """Do now what launches on `device` would do on first use (shared-memory
        opt-in of every kernel, the stream-K workspaces), e.g. before a stream capture."""
        if self._prepare(device) != OG_OK:
            raise RuntimeError(self.error())

    def tile_order(self, g):
        """The (M index, N index) of every output tile of a bound GEMM, in the order the grid visits them."""
        tiles = self.plan(g)["tiles"]
        buffer = (c_int32 * (2 * tiles))()
        count = self._tile_order(byref(g), buffer, 2 * tiles)
        if count < 0:
            raise RuntimeError(self.error())
        return [(buffer[2 * i], buffer[2 * i + 1]) for i in range(count)]

    def test_overcredit_next_launch(self, nbytes):
        """Testing aid: the calling thread's next launch credits `nbytes` more to every
        stage barrier than its loads deliver, so its first wait for data runs out."""
        self._overcredit(int(nbytes))

    def plan(self, g, device=-1):
        out = OgPlan()
        if self._plan(byref(g), device, byref(out)) != OG_OK:
            raise RuntimeError(self.error())
        return {name: getattr(out, name) for name, _ in OgPlan._fields_}

    def describe(self, g, sm_count=148):
        """Every field of the tile plan of a bound OgGemm, as a dict of ints."""
        import json

        text = ctypes.create_string_buffer(2048)
        if self._describe(byref(g), sm_count, text, len(text)) != OG_OK:
            raise RuntimeError(self.error())
        return json.loads(text.value.decode())

    def quantize(self, name, x, packed, scales, blocked):
        """Run the quantisation kernel on CUDA tensors (`scales` / `blocked` may be None)."""
        device = x.get_device()
        status = self._quantize(
            name.encode(), x.data_ptr(), int(x.dtype is torch.float32), x.size(0), x.size(1), packed.data_ptr(),
            0 if scales is None else scales.data_ptr(), 0 if blocked is None else blocked.data_ptr(),
            device, raw_stream(device),
        )
        if status != OG_OK:
            raise RuntimeError(self._quantize_error().decode())

    def set_independent_inputs(self, yes):
        """Vouch (or stop vouching) that no earlier kernel of the stream writes a launch's
        operands.  Process-wide; returns the previous setting, so a tool that turns it on
        for its own loop can put it back."""
        global _independent_inputs
        before, _independent_inputs = _independent_inputs, bool(yes)
        self._independent(int(bool(yes)))
        return before

    def set_fixed_kernels(self, yes):
        """Let launches use the kernels compiled for one tile shape (default), or send all to the run-time kernel."""
        self._fixed(int(bool(yes)))

    def set_wait_limit_ms(self, ms):
        self._set_limit(int(ms))


_libraries, _lock = {}, threading.Lock()
_independent_inputs = False  # mirror of the library's process-wide switch


def independent_inputs():
    """The setting `Library.set_independent_inputs` last made in this process (default off)."""
    return _independent_inputs


def library(impl):
    """The loaded library for `impl`, loading it on first use."""
    with _lock:
        if impl not in _libraries:
            _libraries[impl] = Library(impl)
    return _libraries[impl]


def bind(name, m, n, k, config):
    """`(library, OgGemm)` for a configuration on a shape."""
    lib = library(lookup(name).impl)
    return lib, lib.bind(name, m, n, k, config)
