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

One addition to the schema: an entry may carry `config_dependent` (and
`measured_dependent`) beside `config`.  The reference's kernels never wait for
the previous kernel of the stream before they load (its launches always
overlap, opengemm/src/mm/kernel.cuh:209,479-483), so its one configuration per
shape is the best for back-to-back launches of independent GEMMs.  Here that
is a mode the caller opts into (`og_b200_set_independent_inputs`); by default
a launch's loads wait for the previous kernel, as a chain of dependent GEMMs
needs.  The two modes want different plans wherever a GEMM has fewer tiles
than the GPU has SMs: independent launches run side by side, so a few fat CTAs
win; a dependent launch has the GPU to itself and wants every SM it can use.
`config` is the former (what the reference's schema means), `config_dependent`
the latter, stored only where tuning found it to differ.
"""

import json
import os
import re
from pathlib import Path

from .dtypes import DTYPES, sf_block
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


# Formats that run the same kernel instantiation on operands of the same width
# in shared memory (csrc/plan.h FORMATS: MMA kind and container bits), so that a
# configuration tuned for one is the right one for the others.
KERNEL_FAMILIES = (
    ("bf16", "f16"),
    ("s8", "u8"),
    ("e4m3", "e5m2", "e4m3xe5m2", "e3m2", "e2m3", "e2m1"),
)


def sibling_entry(name, m, n, k):
    """The stored entry of a format of `name`'s kernel family for this shape
    (the first member that has a usable one), or None."""
    for family in KERNEL_FAMILIES:
        if name in family:
            for other in family:
                if other != name:
                    entry = stored_entry(other, m, n, k)
                    if entry is not None and entry.get("config") is not None:
                        return entry
    return None


def _round_up(x, to):
    return -(-x // to) * to


# Constants of the tile-time model below, fitted to measurements on B200.  A K
# block (128 bytes of K per row) keeps the tensor pipe busy for 2 x tile_n SM
# clocks; L2 feeds an SM's ring about 80 bytes per clock when every SM pulls at
# once; the output leaves at the SM's share of HBM write bandwidth.  A long
# tensor-bound kernel runs into the board's power limit, which holds the SM
# clock near 1.35 GHz however the tiles are spread over the SMs, while a
# critical path (the waves) runs at up to 1.9 GHz: a partly idle last wave
# costs less than its share of tiles suggests.
LOAD_BYTES_PER_CLOCK = 80.0
STORE_BYTES_PER_CLOCK = 27.0
DRAIN_CLOCKS = 2000.0   # single-accumulator tiles: the MMA warp waits while tensor memory is read out
TILE_CLOCKS = 1200.0    # hand-offs per tile that nothing overlaps
PAIR_CLOCKS = 400.0     # more of them when two CTAs share a tile (barriers across the pair)
TRAFFIC_ENERGY = 0.25   # energy of moving a clock's worth of operand bytes, in tensor-pipe clocks
BOOST_GHZ, CAPPED_GHZ = 1.9, 1.35
HBM_BYTES_PER_US = 6.5e6
HBM_SATURATING_CTAS = 128.0
LAUNCH_FLOOR_US = 4.0   # back-to-back launches of one tile take about this long each
CTA_US = 0.004          # what a CTA costs the launches around it (ties go to fewer, fatter CTAs)
PAIR_FROM_US = 9.0      # below this a pair's set-up (cluster synchronisation, both CTAs' tensor memory) shows ...
PAIR_SETUP_US = 1.0     # ... as about this much


def _smem_bytes_per_value(name):
    d = DTYPES[name]
    if d.impl == "smm":
        return 0.5 if d.bits == 4 else 1.0
    return max(1.0, d.bits / 8)  # dense sub-byte values are unpacked to bytes by the tensor map


def modelled_us(name, m, n, k, use_2cta, output_n, swap_ab, dependent=False):
    """Estimated microseconds for one GEMM with the given tiling: the slower
    of the critical path (waves x tile time at the boost clock, the K loop
    bound by the tensor pipe or by L2 -> shared-memory traffic) and the
    power-limited time of all tiles' work spread over the SMs.  `dependent`:
    the launch does not overlap its neighbours, so a long kernel's waves run
    at the power-limited clock one after the other (a partly filled last wave
    then costs a whole tile time: mxfp8 2048x2048x14336 on 88 tiles of 256x192
    takes 49 us per launch overlapping and 74 us alone)."""
    d = DTYPES[name]
    scaled = d.impl == "smm"
    rows_m, rows_n = (n, m) if swap_ab else (m, n)
    cg = 2 if use_2cta else 1
    block_k = 128 / _smem_bytes_per_value(name)
    k_blocks = -(-k // int(block_k))
    scale_bytes = 0.0
    if scaled:
        atoms = block_k / (4 * sf_block(d))
        scale_bytes = atoms * 512 * (1 + (2 if output_n > 128 else 1))
    slots = SM_COUNT // cg
    tiles = -(-rows_m // (128 * cg)) * -(-rows_n // output_n)
    waves = -(-tiles // slots)
    compute = 2.0 * output_n
    load = ((128 + output_n / cg) * 128 + scale_bytes) / LOAD_BYTES_PER_CLOCK
    store = 128 * output_n * d.out.itemsize / STORE_BYTES_PER_CLOCK
    extra = TILE_CLOCKS + (PAIR_CLOCKS if use_2cta else 0.0) + (DRAIN_CLOCKS if scaled and output_n > 192 else 0.0)
    tile = max(k_blocks * max(compute, load), store) + extra
    energy = max(k_blocks * (compute + TRAFFIC_ENERGY * load), store) + extra
    power_us = tiles / slots * energy / (CAPPED_GHZ * 1e3)
    path_us = waves * tile / ((CAPPED_GHZ if dependent and power_us > 15.0 else BOOST_GHZ) * 1e3)
    # Operands and output cross HBM at least once; few CTAs cannot keep enough
    # loads in flight to saturate it.
    hbm_bytes = (m * k + n * k) * d.bits / 8 + m * n * d.out.itemsize
    streams = min(1.0, min(tiles, slots) * cg / HBM_SATURATING_CTAS)
    hbm_us = hbm_bytes / (HBM_BYTES_PER_US * streams)
    return max(path_us, power_us, hbm_us) + store / (BOOST_GHZ * 1e3)


def heuristic_config(name, m, n, k, dependent=False):
    """A configuration chosen by rule, for shapes nothing is stored for.

    Small M rides the MMA's N side (swap_ab) so the 128-row side streams B.
    Pair size and tile width minimise `modelled_us`; estimates within 2 %
    go to the pair and the wider tile (less operand traffic).  `dependent`:
    for launches that wait for the previous kernel (the default mode), where
    nothing is gained by leaving SMs to the neighbouring launches.
    """
    d = DTYPES[name]
    scaled = d.impl == "smm"
    if scaled and d.bits == 4 and m <= 64 and n >= 1024 and not dependent:
        # Block-scaled fp4 decode (tuned on 1..64 x 7168..57344 x 8192): 128 x 256 tiles
        # on single CTAs, M on the padded 128-row side (rows past M are TMA zero fill and
        # cost no traffic).  Few fat CTAs let consecutive launches run side by side.
        return _with_defaults({"use_2cta": False, "output_n": 256, "swap_ab": False, "supergroup": 1}, scaled)
    if scaled and m <= 64 and n >= 1024 and dependent:
        # A block-scaled decode launch with the GPU to itself (tuned on 1..64 x 2048..14336):
        # M on the padded 128-row side again, tiles narrow enough to put a CTA on most SMs.
        width = 64 if n < 11264 else 128 if n < 28672 else 256
        return _with_defaults({"use_2cta": False, "output_n": width, "swap_ab": False, "supergroup": 8}, scaled)
    swap = m <= 64 and n >= 2 * m
    rows_m, rows_n = (n, m) if swap else (m, n)
    # Widths that fill whole 128-byte lines of the staged rows.
    step = 64 if (scaled or d.out.itemsize == 2) else 32
    cap = _round_up(rows_n, 16)
    if scaled and cap >= 64:
        cap = _round_up(cap, 64)
    widths = [w for w in range(step, 257, step) if w <= cap]
    if cap <= 256 and cap not in widths and (not scaled or cap < 64):
        widths.append(cap)  # one tile spanning all of a narrow N
    widths.sort()
    best = None
    for two in (True, False):
        if two and rows_m <= 128:
            continue
        for width in reversed(widths):
            if two and width < 32:
                continue
            cost = modelled_us(name, m, n, k, two, width, swap, dependent)
            # Measured corrections to the model: an overlapping launch is never shorter
            # than the launch floor, below which fewer CTAs win (consecutive launches
            # then run side by side); a short kernel loses about a microsecond to a
            # pair's set-up.
            ctas = -(-rows_m // (256 if two else 128)) * -(-rows_n // width) * (2 if two else 1)
            if not dependent:
                cost = max(cost, LAUNCH_FLOOR_US) + CTA_US * min(ctas, SM_COUNT)
            if two and cost < PAIR_FROM_US:
                cost += PAIR_SETUP_US  # single CTAs won 90 % of the tuned shapes that run under 9 us
            if best is None or cost < best[0] * 0.98:
                best = (cost, two, width)
    _, use_2cta, output_n = best
    return _with_defaults({"use_2cta": bool(use_2cta), "output_n": int(output_n), "swap_ab": bool(swap), "supergroup": 8},
                          scaled)


def _with_defaults(knobs, scaled):
    """A complete configuration in the store's schema from the knobs the heuristic decides."""
    config = {
        "use_2cta": bool(knobs["use_2cta"]),
        "output_n": int(knobs["output_n"]),
        "use_clc": False,
        "supergroup": int(knobs["supergroup"]),
        "swap_ab": bool(knobs["swap_ab"]),
        "epi_direct": 0,
        "cluster_m": 2 if knobs["use_2cta"] else 1,
        "cluster_n": 1,
        "cluster_k": 1,
    }
    if scaled:
        config.update({"epi_trade": 0, "deep_stages": 0, "persistent": 1})
    else:
        config.update({"block_m": 128, "stages": 0, "epi_hold": 1, "epi_double": 0, "split_k": 1,
                       "walk": 0, "l2_promo": 0})
    return config


def independent_mode():
    """Whether this process has told the library that launches' inputs are independent."""
    from . import capi

    return capi.independent_inputs()


def planned_ctas(config, m, n):
    """CTAs a configuration launches for an M x N output (at most one per SM)."""
    rows_m, rows_n = (n, m) if config.get("swap_ab") else (m, n)
    pair = 2 if config.get("use_2cta") else 1
    return min(SM_COUNT, -(-rows_m // (128 * pair)) * -(-rows_n // max(16, int(config["output_n"]))) * pair)


def config_of(entry, dependent):
    """The configuration of a stored entry for the launch mode.  An entry tuned
    only for overlapping launches whose plan leaves most of the GPU idle is
    passed over, for a dependent launch, when the rule for dependent launches
    would put a third as many CTAs again to work (on the shapes tuned both ways
    that rule chose at least 0.6 of the tuned CTA count every time)."""
    if dependent and entry.get("config_dependent") is not None:
        return entry["config_dependent"]
    config = entry["config"]
    if dependent and config is not None:
        m, n = entry["m"], entry["n"]
        used = planned_ctas(config, m, n)
        if used < 100:
            ruled = heuristic_config(entry["dtype"], m, n, entry["k"], dependent=True)
            if planned_ctas(ruled, m, n) >= max(16, 1.3 * used):  # a handful of CTAs either way: launch-bound, leave it
                return ruled
    return config


def resolve_config(name, m, n, k, dependent=None):
    """The configuration for a (dtype, shape): stored, else tuned now when
    OPENGEMM_AUTOTUNE=1, else what is stored for a format of the same kernel
    family (`KERNEL_FAMILIES`), else the heuristic.  `dependent` picks between
    an entry's two configurations (default: by the library's current mode).

    Raises:
        ValueError: if the shape is recorded as unimplementable.
    """
    if dependent is None:
        dependent = not independent_mode()
    entry = stored_entry(name, m, n, k)
    if entry is None:
        if os.environ.get("OPENGEMM_AUTOTUNE") == "1":
            from .tune import tune

            log(f"no stored configuration for {name} {m}x{n}x{k}; tuning it now")
            return tune(name, m, n, k, dependent=dependent)
        entry = sibling_entry(name, m, n, k)
        if entry is not None:
            return config_of(entry, dependent)
        return heuristic_config(name, m, n, k, dependent)
    if entry.get("config") is None:
        why = entry.get("unimplementable", "recorded as unimplementable")
        raise ValueError(f"{name} {m}x{n}x{k} cannot be served: {why}")
    return config_of(entry, dependent)


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
