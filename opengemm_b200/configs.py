"""Stored configurations: the shipped ones, what tuning adds, and a heuristic.

Same store and schema as the reference (opengemm/python/configs.py:15-105):
a JSON file `{"kind"?, "arch": "sm_100", "entries": [{dtype, m, n, k,
config | null, unimplementable?, measured?}]}`; the local store
(`$OPENGEMM_CONFIGS/tuned_configs.json`, else `./opengemm-configs/`) wins over
the shipped files; writes are serialised by a lock file and land by atomic
rename.  Files written by the reference load unchanged.

Where the reference tunes on the spot when nothing is stored
(configs.py:63-80), this build answers from `heuristic_config` unless
OPENGEMM_AUTOTUNE=1 asks for a sweep, so an untuned shape costs no GPU minutes.
"""

import json
import os
import re
from pathlib import Path

from .dtypes import DTYPES
from .log import log

PACKAGE = Path(__file__).resolve().parent
TUNED_DIR = "opengemm-configs"
TUNED_FILE = "tuned_configs.json"
SM_COUNT = 148


def load_shapes():
    """Distinct (M, N, K) triples of shapes.jsonc, in file order."""
    path = PACKAGE / "shapes.jsonc"
    if not path.exists():
        return []
    text = re.sub(r"//[^\n]*", "", path.read_text())
    return list(dict.fromkeys(tuple(shape) for shape in json.loads(text)))


def tuned_path():
    """Where new tunings are written."""
    directory = os.environ.get("OPENGEMM_CONFIGS")
    return (Path(directory) if directory else Path.cwd() / TUNED_DIR) / TUNED_FILE


def config_path(impl):
    """The configurations shipped with the package."""
    return PACKAGE / "configs" / f"{impl}.json"


def entry_key(entry):
    return (entry["dtype"], entry["m"], entry["n"], entry["k"])


def _entries(path):
    try:
        return json.loads(Path(path).read_text())["entries"]
    except FileNotFoundError:
        return []


def tuned_entries(impl=None):
    return [e for e in _entries(tuned_path()) if impl is None or DTYPES[e["dtype"]].impl == impl]


def stored_entries(impl):
    """Every entry for `impl`; the local store shadows the shipped file."""
    merged = {entry_key(e): e for e in _entries(config_path(impl))}
    merged.update({entry_key(e): e for e in tuned_entries(impl)})
    return list(merged.values())


def load_configs(impl, dtype=None):
    return {
        entry_key(e): e["config"]
        for e in stored_entries(impl)
        if e.get("config") is not None and (dtype is None or e["dtype"] == dtype)
    }


def stored_entry(name, m, n, k):
    """The stored entry for (dtype, shape), local store first; None when there is none."""
    impl = DTYPES[name].impl
    for entries in (tuned_entries(impl), _entries(config_path(impl))):
        for e in entries:
            if entry_key(e) == (name, m, n, k):
                return e
    return None


def _round_up(x, to):
    return -(-x // to) * to


def heuristic_config(name, m, n, k):
    """A configuration chosen by rule, for shapes nothing is stored for.

    Small M rides the MMA's N side (swap_ab) so the 128-row side streams B;
    pairs of CTAs take 256-row tiles once there are enough of them to fill the
    GPU; the tile width is the widest the format allows, narrowed when that
    wastes less of the last wave of 148 SMs.
    """
    d = DTYPES[name]
    scaled = d.impl == "smm"
    swap = m <= 64 and n >= 2 * m
    rows_m, rows_n = (n, m) if swap else (m, n)
    step = 64 if scaled else 16
    widest = 256 if not scaled else 192
    if rows_n <= widest:
        output_n = max(16, _round_up(rows_n, 16))
        if scaled and not (output_n < 64):
            output_n = _round_up(output_n, 64)
    else:
        best = None
        for cand in range(widest, 63, -step):
            for two in (1, 0):
                tile_m = 256 if two else 128
                tiles = -(-rows_m // tile_m) * -(-rows_n // cand)
                slots = SM_COUNT // (2 if two else 1)
                waves = -(-tiles // slots)
                # time ~ waves x tile work; prefer pairs (less operand traffic) on ties
                cost = waves * tile_m * cand / (2 if two else 1) * (1.0 if two else 1.04)
                if best is None or cost < best[0] - 1e-9:
                    best = (cost, cand, two)
        output_n = best[1]
    tiles_pair = -(-rows_m // 256) * -(-rows_n // output_n)
    use_2cta = int(rows_m >= 256 and output_n >= 32 and tiles_pair >= SM_COUNT // 4)
    if rows_n > widest:
        use_2cta = int(best[2] and rows_m >= 256)
    config = {
        "use_2cta": bool(use_2cta),
        "output_n": int(output_n),
        "use_clc": False,
        "supergroup": 8,
        "swap_ab": bool(swap),
        "epi_direct": 0,
        "cluster_m": 2 if use_2cta else 1,
        "cluster_n": 1,
        "cluster_k": 1,
    }
    if scaled:
        config.update({"epi_trade": 0, "deep_stages": 0, "persistent": 1})
    else:
        config.update({"block_m": 128, "stages": 0, "epi_hold": 1, "epi_double": 0, "split_k": 1,
                       "walk": 0, "l2_promo": 0})
    return config


def resolve_config(name, m, n, k):
    """The configuration for a (dtype, shape): stored, else tuned now when
    OPENGEMM_AUTOTUNE=1, else the heuristic.

    Raises:
        ValueError: if the shape is recorded as unimplementable.
    """
    entry = stored_entry(name, m, n, k)
    if entry is None:
        if os.environ.get("OPENGEMM_AUTOTUNE") == "1":
            from .tune import tune

            log(f"no stored configuration for {name} {m}x{n}x{k}; tuning it now")
            return tune(name, m, n, k)
        return heuristic_config(name, m, n, k)
    if entry.get("config") is None:
        why = entry.get("unimplementable", "recorded as unimplementable")
        raise ValueError(f"{name} {m}x{n}x{k} cannot be served: {why}")
    return entry["config"]


def write_entry(impl, entry):
    """Store `entry` in the local store, replacing any entry for the same
    (dtype, shape).  Serialised through a lock file; lands by atomic rename;
    entries stay sorted by dtype, then by shapes.jsonc order.  Returns the path."""
    path = tuned_path()
    path.parent.mkdir(parents=True, exist_ok=True)
    with (path.parent / ".tuned_configs.lock").open("w") as lock_file:
        os.lockf(lock_file.fileno(), os.F_LOCK, 0)
        try:
            store = json.loads(path.read_text())
        except FileNotFoundError:
            store = {"arch": "sm_100", "entries": []}
        shape_rank = {shape: i for i, shape in enumerate(load_shapes())}
        dtype_rank = {name: i for i, name in enumerate(DTYPES)}
        kept = [e for e in store["entries"] if entry_key(e) != entry_key(entry)] + [entry]
        kept.sort(key=lambda e: (dtype_rank.get(e["dtype"], 1 << 30),
                                 shape_rank.get((e["m"], e["n"], e["k"]), 1 << 30),
                                 e["m"], e["n"], e["k"]))
        store["entries"] = kept
        scratch = path.with_suffix(".json.tmp")
        scratch.write_text(json.dumps(store, indent=1) + "\n")
        scratch.replace(path)
    return path
