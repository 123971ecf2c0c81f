"""Measure every format over the whole shape suite, each (format, shape) with
the configuration `gemm()` would dispatch, against torch's library kernel for
that format, and check every result against the reference product.

    python -m opengemm_b200.benchmark                          # 14 formats x shapes.jsonc
    python -m opengemm_b200.benchmark --dtype bf16 e4m3 nvfp4
    python -m opengemm_b200.benchmark --shape 4096 4096 4096
    python -m opengemm_b200.benchmark --quick                  # short timing windows
    python -m opengemm_b200.benchmark --tune-missing           # tune shapes with no stored entry first

Counterpart of the reference's suite runner (scripts/benchmark.py:1-60): the
same harness on both sides (rotating operand sets larger than twice L2, CUDA
events around back-to-back launches, medians of windows), a JSON report, and a
non-zero exit status if any result is incorrect or fails to launch, so the run
doubles as a regression test.  One difference: a shape with no stored entry is
measured with the heuristic configuration `gemm()` falls back to (and marked
`heuristic`) instead of being skipped.  Formats torch has no kernel for (u8,
e5m2, e3m2, e2m3, e2m1, mxfp4) are compared, as in the reference
(scripts/benchmark.py:90-119), with the fastest correct configuration of the
CUTLASS stand-in library when `--cutlass DIR` (default oracle/_ref) holds one.
"""

import argparse
import json
import math
import statistics
import sys
import time
from pathlib import Path

import torch

from . import capi, configs, harness
from .dtypes import DTYPES
from .log import log

LOW_SPEEDUP = 0.95


def cutlass_baseline(directory, buffers, name, m, n, k, window_ms):
    """The fastest CUTLASS configuration that reproduces the reference product:
    `(callable, tile label)`, or `(None, reason)`.  Every configuration is
    checked before it is timed, so a baseline that computes the wrong thing
    cannot flatter the kernel compared with it."""
    from . import compare

    if directory is None or compare.cutlass_baselines(directory) is None:
        return None, "no CUTLASS comparator built"
    want = harness.reference(buffers[0], name)
    rtol, atol = harness.tolerance(name, k)
    best, wrong = None, []
    checks = dict(compare.cutlass_runners(directory, name, m, n, k, buffers[:1]))
    for tile, call in compare.cutlass_runners(directory, name, m, n, k, buffers):
        try:
            out = checks[tile]()
            torch.cuda.synchronize()
            torch.testing.assert_close(out, want, rtol=rtol, atol=atol)
            us = harness.timed(call, window_ms=min(window_ms, 20.0), repeats=1)
        except Exception as exc:
            wrong.append(f"{tile}: {str(exc).splitlines()[0][:60]}")
            continue
        if best is None or us < best[0]:
            best = (us, call, tile)
    if best is None:
        return None, ("no CUTLASS configuration for this format" if not wrong else "no CUTLASS tile worked: " + "; ".join(wrong))
    return best[1], best[2]


def measure(name, m, n, k, window_ms, tune_missing=False, cutlass=None):
    """One row of the report."""
    row = {"dtype": name, "m": m, "n": n, "k": k}
    stored = configs.stored_entry(name, m, n, k)
    if stored is None and tune_missing:
        from . import tune

        try:
            tune.tune(name, m, n, k)
            stored = configs.stored_entry(name, m, n, k)
        except RuntimeError as exc:
            row["status"] = f"skipped: {str(exc)[:100]}"
            return row
    dependent = not configs.independent_mode()
    config = configs.config_of(stored, dependent) if stored else configs.resolve_config(name, m, n, k, dependent)
    row["source"] = "stored" if stored else "heuristic"
    row["launches"] = "dependent" if dependent else "independent"
    try:
        bound = capi.bind(name, m, n, k, config)
    except RuntimeError as exc:
        row["status"] = f"skipped: {str(exc)[:100]}"  # e.g. K not a multiple the format accepts
        return row
    buffers = harness.make_input_set(m, n, k, name, cap_bytes=8 << 30)
    wrong = harness.correctness_error(buffers, bound, name, k)
    if wrong:
        row["status"] = f"INCORRECT: {wrong}"
        return row
    kernel = harness.runner(buffers, bound)
    baseline, why = harness.baseline_for(buffers, name)
    baseline_kind = "library"
    if baseline is None:
        baseline, tile_or_why = cutlass_baseline(cutlass, buffers, name, m, n, k, window_ms)
        if baseline is not None:
            baseline_kind = f"cutlass {tile_or_why}"
        elif cutlass is not None:
            why = f"{why}; {tile_or_why}"
    # Windows of the two sides alternate, so that clock and temperature drift
    # on a power-capped GPU falls on both alike; medians of three each.
    ours, theirs = [], []
    for _ in range(3):
        ours.append(harness.timed(kernel, window_ms=window_ms, repeats=1))
        if baseline:
            theirs.append(harness.timed(baseline, window_ms=window_ms, repeats=1))
    us = statistics.median(ours)
    flops = 2.0 * m * n * k
    plan = bound[0].plan(bound[1])
    row.update(status="ok", us=round(us, 3), tflops=round(flops / us / 1e6, 2),
               gbs=round(harness.iteration_bytes(name, m, n, k) / us / 1e3, 1),
               tile=f"{plan['tile_m']}x{plan['tile_n']}")
    if baseline:
        base = statistics.median(theirs)
        row.update(baseline_us=round(base, 3), speedup=round(base / us, 3), baseline_kind=baseline_kind)
    else:
        row["baseline"] = why
    return row


def summarise(rows):
    """Per format: rows measured, geometric-mean speed-up over the library
    kernel, and how many shapes fall below LOW_SPEEDUP."""
    out = {}
    for name in dict.fromkeys(r["dtype"] for r in rows):
        mine = [r for r in rows if r["dtype"] == name]
        ok = [r for r in mine if r.get("status") == "ok"]
        ratios = [r["speedup"] for r in ok if "speedup" in r]
        out[name] = {
            "measured": len(ok),
            "skipped": sum(1 for r in mine if r.get("status", "").startswith("skipped")),
            "incorrect": sum(1 for r in mine if r.get("status", "").startswith("INCORRECT")),
            "geomean_speedup": round(math.exp(sum(map(math.log, ratios)) / len(ratios)), 3) if ratios else None,
            "below_0.95": sum(1 for x in ratios if x < LOW_SPEEDUP),
        }
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--dtype", nargs="+", default=list(DTYPES), choices=list(DTYPES))
    ap.add_argument("--shape", nargs=3, type=int, metavar=("M", "N", "K"))
    ap.add_argument("--quick", action="store_true", help="10 ms timing windows instead of 100 ms")
    ap.add_argument("--tune-missing", action="store_true")
    ap.add_argument("--cutlass", default=str(Path(__file__).resolve().parents[1] / "oracle" / "_ref"),
                    help="folder holding libcutlass_ref.so, the CUTLASS stand-in baselines (skipped when absent)")
    ap.add_argument("--output", default=None, help="JSON report (default results/perf_<gpu>_<date>.json)")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("the benchmark needs a CUDA device")

    shapes = [tuple(args.shape)] if args.shape else configs.load_shapes()
    window_ms = 10.0 if args.quick else 100.0
    rows, started = [], time.time()
    for name in args.dtype:
        for m, n, k in shapes:
            try:
                row = measure(name, m, n, k, window_ms, args.tune_missing, cutlass=args.cutlass)
            except Exception as exc:  # a failed launch is a result, not the end of the sweep
                row = {"dtype": name, "m": m, "n": n, "k": k, "status": f"FAILED: {str(exc).splitlines()[0][:120]}"}
            rows.append(row)
            tail = ""
            if row.get("status") == "ok":
                tail = f"{row['us']:10.2f} us {row['tflops']:9.1f} TFLOP/s {row['gbs']:8.1f} GB/s  {row['tile']:>8s} {row['source']:9s}"
                tail += f" {row['speedup']:.3f}x" if "speedup" in row else "  no baseline"
            log(f"{name:10s} {m:6d} {n:6d} {k:6d}  {row.get('status', ''):s} {tail}")
            torch.cuda.empty_cache()

    summary = summarise(rows)
    for name, s in summary.items():
        log(f"{name:10s} measured {s['measured']:3d}  skipped {s['skipped']:2d}  incorrect {s['incorrect']}  "
            f"geomean vs library {s['geomean_speedup']}  below {LOW_SPEEDUP}: {s['below_0.95']}")
    stamp = harness.env_stamp()
    path = Path(args.output or f"results/perf_{stamp['gpu'].replace(' ', '_')}_{stamp['date']}.json")
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps({"env": stamp, "seconds": round(time.time() - started, 1), "summary": summary,
                                "rows": rows}, indent=1))
    log(f"report written to {path}")
    bad = [r for r in rows if r.get("status", "").startswith(("INCORRECT", "FAILED"))]
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
