"""Time this library against another shared library that exports the same C
ABI - in practice the reference's own sm_100a kernel libraries, whose twelve
`og_mm_*` / `og_smm_*` entry points (opengemm/src/mm/capi.cu:6-32,
opengemm/src/smm/capi.cu:6-32) this library mirrors - on the same device
buffers, in timing windows that alternate between the two so both meet the
same clocks and temperature.

    python -m opengemm_b200.compare --dir oracle/_ref --dtype e4m3 --shape 4096 4096 4096

`--dir` holds `libopengemm_mm.so`, `libopengemm_smm.so` and
`reference_configs.json` (the other library's stored configurations, in the
configs.json schema); oracle/build_reference_kernels.py produces all three
from a reference checkout.  This is a measuring tool: nothing on the product
path loads another library.
"""

import argparse
import itertools
import json
import math
from pathlib import Path

import torch

from . import capi, harness
from .configs import resolve_config
from .dtypes import DTYPES


def reference_libraries(directory):
    """Paths of the other build's libraries and stored configurations under
    `directory`, or None when any of them is missing."""
    directory = Path(directory)
    found = {"mm": directory / "libopengemm_mm.so", "smm": directory / "libopengemm_smm.so",
             "configs": directory / "reference_configs.json"}
    return found if all(p.exists() for p in found.values()) else None


def nearest_entry(entries, name, m, n, k):
    """The stored entry of `name` for this shape, else the one closest to it in
    log-shape distance (a reference build ships entries for its own shape
    list only).  Returns (entry, exact?) or (None, False)."""
    usable = [e for e in entries if e["dtype"] == name and e.get("config")]
    if not usable:
        return None, False
    distance = lambda e: sum(abs(math.log(x / y)) for x, y in ((e["m"], m), (e["n"], n), (e["k"], k)))
    best = min(usable, key=distance)
    return best, (best["m"], best["n"], best["k"]) == (m, n, k)


_loaded = {}


def other_library(found, impl):
    key = str(found[impl])
    if key not in _loaded:
        _loaded[key] = capi.Library(impl, path=found[impl])
    return _loaded[key]


def interleaved(found, name, m, n, k, sets, ours=None, windows=4, window_ms=60.0, config=None):
    """Microseconds per launch of the other library and of this one on the
    operand/output `sets` (tuples a, b, sfa, sfb, out, rotated), in `windows`
    alternating pairs of timing windows; the order inside a pair flips every
    round.  The two outputs on the first set are compared first."""
    impl = DTYPES[name].impl
    entries = json.loads(Path(found["configs"]).read_text())["entries"]
    entry, exact = nearest_entry(entries, name, m, n, k)
    if entry is None:
        return {"unavailable": f"the other build stores no configuration for {name}"}
    other = other_library(found, impl)
    try:
        g_other = other.bind(name, m, n, k, entry["config"])
    except RuntimeError as exc:
        return {"unavailable": f"the other library does not bind this shape: {str(exc)[:120]}"}
    lib, g = ours if ours is not None else capi.bind(name, m, n, k, config or resolve_config(name, m, n, k))

    def runner(library, bound):
        cycle = itertools.cycle(sets)

        def call():
            a, b, sfa, sfb, out = next(cycle)
            library.launch(bound, a, b, sfa, sfb, out)

        return call

    run_other, run_ours = runner(other, g_other), runner(lib, g)
    a, b, sfa, sfb, out = sets[0]
    other.launch(g_other, a, b, sfa, sfb, out)
    torch.cuda.synchronize()
    theirs = out.clone()
    lib.launch(g, a, b, sfa, sfb, out)
    torch.cuda.synchronize()
    difference = (out.double() - theirs.double()).abs().max().item()
    del theirs

    for fn in (run_other, run_ours):
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    guess = max(harness.elapsed_us(run_ours, 5), 0.5)
    iterations = int(max(5, min(4000, window_ms * 1e3 / guess)))
    times = {"ref": [], "ours": []}
    for round_ in range(windows):
        order = ("ref", "ours") if round_ % 2 == 0 else ("ours", "ref")
        for who in order:
            times[who].append(harness.elapsed_us(run_other if who == "ref" else run_ours, iterations))
    # the first pair of windows also warms the GPU up to its steady clocks: medians over the rest
    settled = {who: (series[1:] if len(series) > 1 else series) for who, series in times.items()}
    ref_us = sorted(settled["ref"])[len(settled["ref"]) // 2]
    ours_us = sorted(settled["ours"])[len(settled["ours"]) // 2]
    return {
        "ref_us": round(ref_us, 2), "ours_us": round(ours_us, 2), "speed_vs_reference_kernel": round(ref_us / ours_us, 3),
        "windows_ref_us": [round(x, 2) for x in times["ref"]], "windows_ours_us": [round(x, 2) for x in times["ours"]],
        "launches_per_window": iterations, "max_abs_difference_of_outputs": difference,
        "reference_config": ("its stored entry for this shape" if exact else
                             f"its stored entry for {entry['m']}x{entry['n']}x{entry['k']} (none for this shape)"),
        "protocol": "alternating windows on the same rotated buffers, CUDA events, median of the windows after the first pair",
    }


# ---- CUTLASS stand-in baselines -------------------------------------------------
#
# For the formats torch has no library kernel for (u8, e5m2, e3m2, e2m3, e2m1,
# mxfp4) the reference's scripts fall back on CUTLASS GEMMs compiled into a small
# library with a C ABI of its own (scripts/utils/cutlass_ref.py:31,54-73,
# scripts/utils/cutlass_ref.cu: ogref_abi / ogref_configs / ogref_config_dtype /
# ogref_config_tile / ogref_launch).  oracle/build_reference_kernels.py --cutlass
# builds that library; this is the wiring that lets the suite runner use it as
# the second baseline.  A comparator only: never loaded by the product path.

CUTLASS_ABI = 1
_cutlass = {}


class CutlassBaselines:
    """`libcutlass_ref.so` through its six `ogref_*` entry points."""

    def __init__(self, path):
        import ctypes
        from ctypes import c_char_p, c_int32, c_void_p

        lib = ctypes.CDLL(str(path))
        lib.ogref_abi.restype = c_int32
        lib.ogref_error.restype = c_char_p
        lib.ogref_configs.restype = c_int32
        lib.ogref_config_dtype.restype, lib.ogref_config_dtype.argtypes = c_char_p, [c_int32]
        lib.ogref_config_tile.restype, lib.ogref_config_tile.argtypes = c_char_p, [c_int32]
        lib.ogref_launch.restype = c_int32
        lib.ogref_launch.argtypes = [c_int32] * 4 + [c_void_p] * 6
        if lib.ogref_abi() != CUTLASS_ABI:
            raise RuntimeError(f"{path} speaks comparator ABI {lib.ogref_abi()}, expected {CUTLASS_ABI}")
        self._lib = lib

    def configs(self, name):
        """`(index, tile label)` of every configuration compiled for format `name`."""
        return [(i, self._lib.ogref_config_tile(i).decode()) for i in range(self._lib.ogref_configs())
                if self._lib.ogref_config_dtype(i).decode() == name]

    def launch(self, index, m, n, k, a, b, sfa, sfb, out):
        status = self._lib.ogref_launch(
            index, m, n, k, a.data_ptr(), b.data_ptr(), 0 if sfa is None else sfa.data_ptr(),
            0 if sfb is None else sfb.data_ptr(), out.data_ptr(), capi.raw_stream(a.get_device()))
        if status != 0:
            raise RuntimeError(self._lib.ogref_error().decode())


def cutlass_baselines(directory):
    """The CUTLASS comparator under `directory`, or None when it was not built."""
    path = Path(directory) / "libcutlass_ref.so"
    if not path.exists():
        return None
    if str(path) not in _cutlass:
        _cutlass[str(path)] = CutlassBaselines(path)
    return _cutlass[str(path)]


def cutlass_runners(directory, name, m, n, k, buffers):
    """`(tile label, callable)` for every CUTLASS configuration of `name` over the
    rotating `buffers` (harness.Inputs); each call returns the output it wrote."""
    library = cutlass_baselines(directory)
    if library is None:
        return []
    out = []
    for index, tile in library.configs(name):
        cycle = itertools.cycle(buffers)

        def call(index=index, cycle=cycle):
            r = next(cycle)
            library.launch(index, m, n, k, r.a, r.b, r.sfa, r.sfb, r.out)
            return r.out

        out.append((tile, call))
    return out


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--dir", required=True, help="folder with the other build's two libraries and reference_configs.json")
    parser.add_argument("--dtype", required=True, choices=sorted(DTYPES))
    parser.add_argument("--shape", nargs=3, type=int, metavar=("M", "N", "K"), action="append", required=True)
    parser.add_argument("--windows", type=int, default=6)
    parser.add_argument("--window-ms", type=float, default=100.0)
    parser.add_argument("--set", dest="overrides", default="{}", help="JSON of configuration keys to override on this library's side")
    args = parser.parse_args()
    found = reference_libraries(args.dir)
    if found is None:
        raise SystemExit(f"{args.dir} does not hold libopengemm_mm.so, libopengemm_smm.so and reference_configs.json")
    capi.library(DTYPES[args.dtype].impl).set_independent_inputs(True)  # the other library overlaps consecutive launches too (this process ends after the comparison)
    for m, n, k in args.shape:
        buffers = harness.make_input_set(m, n, k, args.dtype, cap_bytes=6 << 30)
        sets = [(r.a, r.b, r.sfa, r.sfb, r.out) for r in buffers]
        config = dict(resolve_config(args.dtype, m, n, k), **json.loads(args.overrides))
        result = interleaved(found, args.dtype, m, n, k, sets, windows=args.windows, window_ms=args.window_ms, config=config)
        print(json.dumps({"dtype": args.dtype, "mnk": [m, n, k], **result}), flush=True)
        del buffers, sets
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
