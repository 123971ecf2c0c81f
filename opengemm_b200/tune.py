"""Autotuner for one (dtype, shape): sweep the native tile plans, keep only
candidates that reproduce the reference product, time them, store the winner
in the configs.json format and return it.

Counterpart of the reference's tuner (opengemm/python/tune.py:13-165) with the
same outcome contract - a correctness-gated sweep, ties within 1.5 % going to
the plainer configuration, the winner written with its measurement - over a
different space: because tile width, pair size, operand swap, ring depth,
rasterisation order and band, the tile scheduler (static stride or cluster
launch control), epilogue path and the stream-K schedule are run-time values
here, the sweep is coarse-to-fine (tile geometry first, then pipeline depth,
scheduler and the launch axes around the leaders, the leaders re-timed in
alternation at the end) instead of a walk over precompiled kernels.

Candidates are timed the way the benchmarks time kernels - back-to-back
launches on rotating operand sets that no kernel of the stream writes, so
consecutive launches may overlap (og_b200_set_independent_inputs), as the
reference's launches always do (opengemm/src/mm/kernel.cuh:209,479-483).

    python -m opengemm_b200.tune --dtype e4m3 --shape 4096 4096 4096
"""

import argparse

import torch

from . import capi, harness
from .configs import heuristic_config, load_shapes, stored_entry, write_entry
from .dtypes import DTYPES
from .log import log

TIE = 0.015


def base_config(name, **knobs):
    d = DTYPES[name]
    config = {"use_2cta": False, "output_n": 128, "use_clc": False, "supergroup": 8, "swap_ab": False,
              "epi_direct": 0, "cluster_m": 1, "cluster_n": 1, "cluster_k": 1, "split_k": 1}
    if d.impl == "smm":
        config.update({"epi_trade": 0, "deep_stages": 0, "persistent": 1, "stages": 0, "walk": 0, "l2_promo": 0})
    else:
        config.update({"block_m": 128, "stages": 0, "epi_hold": 1, "epi_double": 0, "walk": 0, "l2_promo": 0})
    config.update(knobs)
    config["cluster_m"] = 2 if config["use_2cta"] else 1
    return config


def geometry_candidates(name, m, n, k):
    """Tile geometries worth timing: pair or single CTA x tile width x operand swap."""
    scaled = DTYPES[name].impl == "smm"
    widths = (64, 128, 192, 256) if scaled else (32, 64, 96, 128, 160, 192, 224, 256)
    out = []
    for swap in ((False, True) if m <= 256 else (False,)):
        rows_m, rows_n = (n, m) if swap else (m, n)
        cap = -(-rows_n // 16) * 16
        fit = sorted({min(w, max(cap, 64 if scaled and rows_n > 32 else 16)) for w in widths} | ({cap} if cap <= 256 and not scaled else set()))
        for two in (True, False):
            if two and rows_m <= 128:
                continue
            for width in fit:
                if rows_n >= 1024 and width < 64:
                    continue
                if two and width < 32:
                    continue
                out.append(base_config(name, use_2cta=two, output_n=int(width), swap_ab=swap))
    return out


def refinements(config, tiles_n, fit_stages=0):
    """Variations around a leading geometry, one axis at a time: rasterisation
    band and order, pipeline depth, the cluster-launch-control scheduler, the
    stream-K split, the epilogue path and L2 promotion."""
    out = []
    for band in sorted({1, 2, 4, 16, tiles_n} - {config["supergroup"]}):
        if 1 <= band <= max(tiles_n, 1):
            out.append(dict(config, supergroup=band))
    if "stages" in config:  # ring depth: the deepest that fits is the default (0)
        for depth in sorted({fit_stages - 1, fit_stages - 2, 4, 3, 2}):
            if 2 <= depth < fit_stages:
                out.append(dict(config, stages=depth))
    out.append(dict(config, use_clc=True))
    out.append(dict(config, split_k=2))
    if not config["use_2cta"]:  # few tiles: let 2, 4 or 8 CTAs of a cluster share each tile along K
        out += [dict(config, cluster_k=ways) for ways in (2, 4, 8)]
    if "walk" in config:
        out += [dict(config, walk=1), dict(config, walk=3)]
    if not config["swap_ab"]:
        out.append(dict(config, epi_direct=1))
    if "l2_promo" in config:
        out.append(dict(config, l2_promo=2))
    return out


def simplicity(config):
    """Sort key under which the plainer configuration wins a tie."""
    return (config["swap_ab"], 0 if config.get("split_k", 1) <= 1 else 1, config.get("cluster_k", 1), int(bool(config.get("use_clc"))),
            config.get("walk", 0), 0 if not config.get("stages") else 1, config.get("epi_direct", 0),
            config.get("l2_promo", 0), int(config["use_2cta"]), config["output_n"], config["supergroup"])


def label(config):
    text = f"v{2 if config['use_2cta'] else 1} n{config['output_n']:<3} sg{config['supergroup']:<2} swap{int(config['swap_ab'])}"
    for key in ("split_k", "cluster_k", "epi_direct", "l2_promo", "stages", "walk", "use_clc"):
        if config.get(key, 0) not in (0, 1, False) or (key in ("epi_direct", "use_clc", "walk") and config.get(key)):
            text += f" {key}{int(config[key])}"
    return text


def merged_entry(existing, name, m, n, k, best, measured, dependent):
    """The store entry after a tuning run: the winner lands in the field of its
    launch mode, whatever the entry holds for the other mode stays."""
    entry = dict(existing or {"dtype": name, "m": m, "n": n, "k": k})
    if dependent:
        entry.update(config_dependent=best, measured_dependent=measured)
        entry.setdefault("config", best)  # the schema's one mandatory configuration
        entry.setdefault("measured", measured)
    else:
        entry.update(config=best, measured=measured)
    return entry


def tune(name, m, n, k, verbose=False, window_ms=15.0, final_ms=60.0, dependent=False):
    """Sweep one (dtype, shape), store the winner and return its configuration.

    `dependent` times the candidates as launches that wait for the previous
    kernel of the stream (the library's default mode) and stores the winner as
    the entry's `config_dependent`, beside whatever `config` it already has;
    otherwise as launches of independent GEMMs, which may overlap, into `config`.

    Raises:
        RuntimeError: if no candidate is correct, or the format cannot take this K.
    """
    impl = DTYPES[name].impl
    library = capi.library(impl)
    # the operand sets below are written once, before any launch; the caller's setting comes back at the end
    independent_before = library.set_independent_inputs(not dependent)
    try:
        return _tune(name, m, n, k, impl, library, verbose, window_ms, final_ms, dependent)
    finally:
        library.set_independent_inputs(independent_before)


def _tune(name, m, n, k, impl, library, verbose, window_ms, final_ms, dependent):
    buffers = harness.make_input_set(m, n, k, name)
    want = harness.reference(buffers[0], name)
    space = geometry_candidates(name, m, n, k)
    log(f"tuning {name} {m}x{n}x{k} on {harness.env_stamp()['gpu']}: {len(space)} tile geometries")

    ranked, rejected, seen = [], 0, set()

    def measure(config):
        nonlocal rejected
        key = tuple(sorted(config.items()))
        if key in seen:
            return
        seen.add(key)
        try:
            bound = capi.bind(name, m, n, k, config)
        except RuntimeError:
            return
        if harness.correctness_error(buffers, bound, name, k, want=want):
            rejected += 1
            return
        us = harness.timed(harness.runner(buffers, bound), window_ms=window_ms)
        ranked.append((us, config))
        if verbose:
            log(f"  {label(config):40s} {us:9.2f} us")

    for config in space:
        measure(config)
    if not ranked:
        raise RuntimeError(f"no correct candidate for {name} {m}x{n}x{k}")
    for _, leader in sorted(ranked, key=lambda row: row[0])[:3]:
        rows_n = m if leader["swap_ab"] else n
        fit = library.plan(capi.bind(name, m, n, k, leader)[1])["stages"]
        for config in refinements(leader, -(-rows_n // leader["output_n"]), fit):
            measure(config)

    # The short windows rank candidates at whatever clocks each happened to
    # meet.  The leaders are timed again in longer windows, in alternation, so
    # all of them see the same warm, power-limited GPU; that ranking decides.
    ranked.sort(key=lambda row: row[0])
    finalists = [config for _, config in ranked[:6]]
    runners = [harness.runner(buffers, capi.bind(name, m, n, k, config)) for config in finalists]
    rounds = [[harness.timed(run, window_ms=final_ms, repeats=1, warmup=1) for run in runners] for _ in range(3)]
    final = sorted((sorted(times)[1], config) for times, config in zip(zip(*rounds), finalists))
    if verbose:
        for us, config in final:
            log(f"  final {label(config):40s} {us:9.2f} us")
    fastest = final[0][0]
    best = min((row for row in final if row[0] <= fastest * (1 + TIE)), key=lambda row: simplicity(row[1]))[1]

    kernel = harness.runner(buffers, capi.bind(name, m, n, k, best))
    us = harness.timed(kernel, window_ms=final_ms, repeats=3)
    baseline, why = harness.baseline_for(buffers, name)
    base = harness.timed(baseline, window_ms=final_ms, repeats=3) if baseline else None
    log(f"best: {label(best)}  ({len(ranked)} timed, {rejected} failed correctness)")
    measured = {"us": round(us, 3), "cublas_us": base and round(base, 3), "env": harness.env_stamp()}
    path = write_entry(impl, merged_entry(stored_entry(name, m, n, k), name, m, n, k, best, measured, dependent))
    if base:
        log(f"kernel {us:.2f}us  cuBLAS {base:.2f}us  {base / us:.3f}x; stored in {path}")
    else:
        log(f"kernel {us:.2f}us  no baseline: {why}; stored in {path}")
    from . import api

    api.forget(name)
    return best


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--dtype", required=True, choices=sorted(DTYPES))
    group = parser.add_mutually_exclusive_group(required=True)
    group.add_argument("--shape", nargs=3, type=int, metavar=("M", "N", "K"))
    group.add_argument("--all", action="store_true", help="every shape in shapes.jsonc")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--dependent", action="store_true",
                        help="tune for launches that wait for the previous kernel (stored as config_dependent)")
    parser.add_argument("--window-ms", type=float, default=15.0, help="timing window of the sweep")
    parser.add_argument("--final-ms", type=float, default=60.0, help="timing window of the closing round among the leaders")
    args = parser.parse_args()
    for m, n, k in [tuple(args.shape)] if args.shape else load_shapes():
        try:
            tune(args.dtype, m, n, k, verbose=args.verbose, window_ms=args.window_ms, final_ms=args.final_ms,
                 dependent=args.dependent)
        except RuntimeError as exc:
            print(exc, flush=True)


if __name__ == "__main__":
    main()
