#!/usr/bin/env python3
"""Benchmark of the GEMM hot path on B200: one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4]

Workload: the largest single-GPU configuration of the baseline, the nvfp4
block-scaled GEMM M = 8192, N = 28672, K = 8192 -> bf16 (operands from
N(0,1), scale = amax/6 as ue4m3 per 16 values).  One step = one GEMM call on
the next of several operand sets (rotated so no step reads what its
predecessor left in L2).  With N > 1 ranks (one per GPU, launched by
torch.distributed.run) the same GEMM is N-sharded: rank r owns rows
shard_bounds(N, ranks, r) of B, of B's scales and the matching columns of C;
A and its scales are replicated; no collective is on the data path.  The job
is the whole GEMM, so scaling is strong: `value` = 2*M*N*K / the slowest
rank's time per step.

`value` times the kernel through the C ABI with operands resident in HBM;
`e2e` times `opengemm_b200.gemm` fed from pinned host memory, with the
host->device copies of the rank's operands and the device->host copy of its
part of C inside the timed region every step.  Before any timing the first
operand set's output is checked against the CPU oracle on sampled rows and
columns; a miss ends the run with a non-zero exit code.  `--impl reference`
times the reference's CPU path (its correctness oracle, a float32 matmul of
the dequantised operands) on the host cores through the numpy port under
oracle/.
"""

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from collections import namedtuple
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# The five configurations of the baseline (and the mixed-fp8 variant of the second).
WORKLOADS = {
    "c1": {"name": "bf16", "m": 1024, "n": 1024, "k": 1024, "what": "bf16 -> f32 GEMM M=N=K=1024, N(0,1)"},
    "c2": {"name": "e4m3", "m": 4096, "n": 4096, "k": 4096,
           "what": "fp8 e4m3 x e4m3 -> f32 GEMM M=N=K=4096, N(0,1)*16 clamped to +-448"},
    "c2m": {"name": "e4m3xe5m2", "m": 4096, "n": 4096, "k": 4096,
            "what": "fp8 e4m3(A) x e5m2(B) -> f32 GEMM M=N=K=4096, B ~ N(0,1)*64 clamped to +-57344"},
    "c3": {"name": "s8", "m": 8192, "n": 8192, "k": 8192, "what": "s8 x s8 -> s32 GEMM M=N=K=8192, uniform [-128,127]"},
    "c4": {"name": "nvfp4", "m": 8192, "n": 28672, "k": 8192,
           "what": "nvfp4 block-scaled GEMM 8192x28672x8192 -> bf16, N(0,1), scale = amax/6 as ue4m3 per 16"},
    "c5": {"name": "mxfp4", "m": 64, "n": 57344, "k": 8192,
           "what": "mxfp4 block-scaled decode GEMM 64x57344x8192 -> bf16, N(0,1), scale = 2^floor(log2(amax/6)) per 32"},
}
HEADLINE = "c4"
SHARDED = ("c3", "c4", "c5")  # the configurations the baseline shards along N
L2_BYTES = 126 * 2**20
SM_COUNT = 148
# Dense tensor-core peaks by format relative to bf16 (nominal bf16 2250 TFLOP/s):
# fp8 / int8 run at twice, fp4 at four times the bf16 rate.
RATE_VS_BF16 = {"bf16": 1.0, "e4m3": 2.0, "e4m3xe5m2": 2.0, "s8": 2.0, "nvfp4": 4.0, "mxfp4": 4.0}
NOMINAL_BF16_TFLOPS = 2250.0
# dram bytes (read + write) of one launch of the dominant kernel in this
# benchmark's own rotation of buffers, from the ncu captures summarised under
# profiles/, keyed by (format, m, n, k); None where no capture is committed.
NCU_TRAFFIC_BYTES = {
    ("nvfp4", 8192, 28672, 8192): 737e6,   # profiles/gemm_kernel_c4_nvfp4_8192x28672x8192.md
    ("e4m3", 4096, 4096, 4096): 52.3e6,    # profiles/gemm_kernel_c2_e4m3_4096.md
    ("mxfp4", 64, 57344, 8192): 252.0e6,   # profiles/gemm_kernel_c5_mxfp4_decode_64x57344x8192.md
}

Operands = namedtuple("Operands", "a b sfa sfb sfa_raw sfb_raw")


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        return {"bf16_burst": peaks["bf16_tflops"], "bf16_sustained": peaks["bf16_tflops_sustained"],
                "hbm_gbs": peaks["hbm_gbs"], "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, begin, end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        inside = [r for t, r in self.rows if begin <= t <= end + 0.2] or [r for _, r in self.rows]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no sample"]}
        def num(x):
            try:
                return float(x)
            except ValueError:
                return float("nan")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({name for r in inside for name, flag in zip(names, r[5:9]) if flag.lower().startswith("active")})
        return {"sm_mhz": statistics.median(num(r[1]) for r in inside), "sm_max_mhz": num(inside[0][2]),
                "power_w": max(num(r[3]) for r in inside), "samples": len(inside), "reasons": reasons}


def quantize_fp4(torch, x, block, power_of_two):
    """Block-scaled e2m1 as the baseline's configurations state it: per `block`
    values along K, scale = amax/6 rounded to ue4m3, or 2^floor(log2(amax/6)) as
    ue8m0 (values beyond +-6 x scale saturate); value/scale to the nearest e2m1,
    two per byte, low nibble first.  Returns (packed, blocked scales, row-major scales)."""
    from opengemm_b200.quant import pack, to_blocked

    rows, k = x.shape
    groups = x.float().reshape(rows, k // block, block)
    scale = (groups.abs().amax(dim=-1, keepdim=True) / 6.0).clamp(min=2.0**-126)
    if power_of_two:
        stored = torch.pow(2.0, torch.floor(torch.log2(scale))).squeeze(-1).to(torch.float8_e8m0fnu)
    else:
        stored = scale.squeeze(-1).to(torch.float8_e4m3fn)
    q = (groups / stored.float().clamp(min=2.0**-126).unsqueeze(-1)).reshape(rows, k).clamp(-6.0, 6.0)
    return pack(q, "e2m1").view(torch.float4_e2m1fn_x2), to_blocked(stored), stored


def make_operands(torch, name, m, n, k, seed, device, seed_b=None):
    """One operand set in the value distribution the baseline names for this
    format, generated on `device` from seeded generators: A from `seed`, B
    from `seed_b` (default: the same generator, after A).  Returns `Operands`;
    the scale fields are None for dense formats, `sf*_raw` are the row-major
    `[rows, K/block]` scales the blocked buffers were built from."""
    g = torch.Generator(device=device).manual_seed(seed)
    gb = g if seed_b is None else torch.Generator(device=device).manual_seed(seed_b)
    if name == "s8":
        a = torch.randint(-128, 128, (m, k), device=device, dtype=torch.int8, generator=g)
        b = torch.randint(-128, 128, (n, k), device=device, dtype=torch.int8, generator=gb)
        return Operands(a, b, None, None, None, None)
    a = torch.randn((m, k), device=device, generator=g)
    b = torch.randn((n, k), device=device, generator=gb)
    if name == "bf16":
        return Operands(a.to(torch.bfloat16), b.to(torch.bfloat16), None, None, None, None)
    if name == "e4m3":
        return Operands((a * 16).clamp(-448, 448).to(torch.float8_e4m3fn),
                        (b * 16).clamp(-448, 448).to(torch.float8_e4m3fn), None, None, None, None)
    if name == "e4m3xe5m2":
        return Operands((a * 16).clamp(-448, 448).to(torch.float8_e4m3fn),
                        (b * 64).clamp(-57344, 57344).to(torch.float8_e5m2), None, None, None, None)
    if name in ("nvfp4", "mxfp4"):
        block, pow2 = (16, False) if name == "nvfp4" else (32, True)
        qa, sfa, raw_a = quantize_fp4(torch, a, block, pow2)
        del a
        qb, sfb, raw_b = quantize_fp4(torch, b, block, pow2)
        return Operands(qa, qb, sfa, sfb, raw_a, raw_b)
    raise KeyError(name)


# ---- the parity gate: sampled rows and columns against the CPU oracle -----------

SAMPLE = 40


def sample_indices(extent, rng, count=SAMPLE):
    """Up to `count` indices: both ends, both sides of every 128 / 256 seam near
    the ends and the middle, the rest random."""
    seams = [0, extent - 1]
    for at in (128, 192, 256, extent // 2 // 128 * 128, (extent - 1) // 256 * 256):
        seams += [at - 1, at]
    picks = [i for i in dict.fromkeys(seams) if 0 <= i < extent]
    spare = count - len(picks)
    if spare > 0 and extent > len(picks):
        picks += list(rng.choice(extent, size=min(spare, extent), replace=False))
    return sorted(set(int(i) for i in picks))[:count]


def raw_rows(torch, t, rows):
    """Selected rows of a device tensor as the storage-typed numpy array the oracle reads."""
    import numpy as np

    index = torch.as_tensor(rows, device=t.device)
    if t.dtype in (torch.float32, torch.int8, torch.uint8):
        return t[index].cpu().numpy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16)[index].cpu().numpy().view(np.uint16)
    return t.view(torch.uint8)[index].cpu().numpy()  # fp8 codes, packed fp4 pairs, scale bytes


def sampled_oracle_check(torch, name, k, ops, out, seed=0):
    """Recompute a sample of output rows x columns of `out` on the CPU oracle
    from the matching rows of A and B (exact for a product whose entries
    depend on one row of each operand) and apply both acceptance rules:
    the reference's assert_close tolerances and the stricter stated bound
    (bit-exact s32; max|x-ref|/max|ref| <= 1e-3 for f32 output; 1 bf16 ulp +
    1e-2 relative for block-scaled output).  Returns a dict for the JSON line."""
    import numpy as np
    from oracle import opengemm_oracle as ora

    m, n = out.shape
    rng = np.random.default_rng(seed + m * 31 + n * 17 + k)
    rows, cols = sample_indices(m, rng), sample_indices(n, rng)
    scaled = ops.sfa_raw is not None
    want = ora.reference(name, raw_rows(torch, ops.a, rows), raw_rows(torch, ops.b, cols),
                         raw_rows(torch, ops.sfa_raw, rows) if scaled else None,
                         raw_rows(torch, ops.sfb_raw, cols) if scaled else None)
    picked = out[torch.as_tensor(rows, device=out.device)][:, torch.as_tensor(cols, device=out.device)].contiguous()
    got = picked.view(torch.int16).cpu().numpy().view(np.uint16) if out.dtype is torch.bfloat16 else picked.cpu().numpy()
    close, worst = ora.check_close(name, k, got, want)
    strict, figure = ora.check_north_star(name, got, want)
    g, w = ora.as_float(name, got), ora.as_float(name, want)
    scale = max(float(np.abs(w).max()), 1e-30)
    result = {"checked": True, "ok": bool(close and strict), "samples": int(got.size),
              "max_rel": float(np.abs(g - w).max() / scale),
              "rule": "sampled rows x columns against the CPU oracle: the reference's assert_close tolerance and "
                      + ("bit-exact s32" if out.dtype is torch.int32 else
                         "max|x-ref|/max|ref| <= 1e-3" if out.dtype is torch.float32 else
                         "|x-ref| <= 1 bf16 ulp + 1e-2 |ref|")}
    if out.dtype is torch.bfloat16:
        result["outputs_needing_the_cancellation_floor"] = int(ora.north_star_floor_users(name, got, want))
    if not result["ok"]:
        result["worst_excess"] = float(worst)
        result["strict_figure"] = float(figure)
    return result


def algorithmic_bytes(name, m, n, k):
    """Bytes one GEMM must move: operands once, output once, scales once
    (the reference's formula, opengemm/python/bench.py:104-109)."""
    from opengemm_b200.dtypes import DTYPES, sf_block

    d = DTYPES[name]
    nbytes = (m * k + n * k) * d.bits // 8 + m * n * d.out.itemsize
    if d.impl == "smm":
        nbytes += (m * k + n * k) // sf_block(d)
    return nbytes


def oracle_inputs(name, rows_a, n, k):
    """Seeded operands for the CPU oracle in the workload's value distribution (numpy)."""
    import numpy as np
    from oracle import opengemm_oracle as ora

    rng = np.random.default_rng(0)
    if name == "s8":
        return (rng.integers(-128, 128, (rows_a, k)).astype(np.int8), rng.integers(-128, 128, (n, k)).astype(np.int8),
                None, None)
    a = rng.standard_normal((rows_a, k), dtype=np.float32)
    b = rng.standard_normal((n, k), dtype=np.float32)
    if name == "bf16":
        return ora.f32_to_bf16(a), ora.f32_to_bf16(b), None, None
    if name == "e4m3":
        return ora.f32_to_e4m3(np.clip(a * 16, -448, 448)), ora.f32_to_e4m3(np.clip(b * 16, -448, 448)), None, None
    if name == "e4m3xe5m2":
        return ora.f32_to_e4m3(np.clip(a * 16, -448, 448)), ora.f32_to_e5m2(np.clip(b * 64, -57344, 57344)), None, None
    # block-scaled: timing only needs valid codes and scales of the right sizes
    block = ora.sf_block(name)
    code = 0x38 if name == "nvfp4" else 127
    return (rng.integers(0, 256, (rows_a, k // 2)).astype(np.uint8), rng.integers(0, 256, (n, k // 2)).astype(np.uint8),
            np.full((rows_a, k // block), code, np.uint8), np.full((n, k // block), code, np.uint8))


def use_all_host_threads():
    """Give the CPU BLAS every host core (launchers such as torch.distributed.run
    export OMP_NUM_THREADS=1, which would cripple the CPU baseline) and return
    the thread count in effect."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        import numpy  # noqa: F401  (loads the BLAS whose pool is resized)
        from threadpoolctl import threadpool_info, threadpool_limits

        threadpool_limits(limits=cores)
        return max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        return 1


def cpu_sample(name, m, n, k, budget_s):
    """Size and time a bounded sample of the workload on the CPU oracle:
    `rows` rows of A against `cols` rows of B (all of K), sized from a probe so
    one pass costs about `budget_s`.  Returns (seconds, rows, cols, runner)."""
    from oracle import opengemm_oracle as ora

    use_all_host_threads()
    rows, cols = min(m, 256), min(n, 4096)
    a, b, sfa, sfb = oracle_inputs(name, rows, cols, k)
    t0 = time.perf_counter()
    ora.reference(name, a, b, sfa, sfb)
    probe = time.perf_counter() - t0
    scale = budget_s / max(probe, 1e-6)
    new_rows = int(max(64, min(m, rows * scale)))
    scale /= new_rows / rows
    new_cols = int(max(256, min(n, cols * max(scale, 1e-3))))
    a, b, sfa, sfb = oracle_inputs(name, new_rows, new_cols, k)
    runner = lambda: ora.reference(name, a, b, sfa, sfb)
    t0 = time.perf_counter()
    runner()
    return time.perf_counter() - t0, new_rows, new_cols, runner


def unit_of(work):
    return ("GB/s", "hbm_gbs") if work["name"] == "mxfp4" and work["m"] <= 128 else ("TFLOP/s", "tflops")


def config_of(work, world):
    """The `config` object of the JSON line; the same for both arms."""
    return {
        "workload": work["what"],
        "m": work["m"], "n": work["n"], "k": work["k"],
        "parallelism": f"nshard{world}" if world > 1 else "1 GPU",
        "sharding": "B, its scales and C split along N on 128-row boundaries, A replicated; no collective",
        "l2": "inputs larger than L2: the GPU arm rotates operand/output sets past 2 x 126 MiB between steps",
    }


def run_reference(args):
    """The reference arm: the reference's CPU path (its oracle) on the host
    cores, through the numpy port, on a bounded sample per step.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    work = WORKLOADS[args.workload]
    name, m, n, k = work["name"], work["m"], work["n"], work["k"]
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    budget = max(0.05, min(2.0, 150.0 / max(args.steps + args.warmup, 1)))
    _, rows, cols, runner = cpu_sample(name, m, n, k, budget)
    for _ in range(args.warmup):
        runner()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        runner()
    seconds = time.perf_counter() - t0
    unit, metric = unit_of(work)
    if unit == "GB/s":
        value = algorithmic_bytes_np(name, rows, cols, k) * args.steps / seconds / 1e9
    else:
        value = 2.0 * rows * cols * k * args.steps / seconds / 1e12
    threads = use_all_host_threads()
    sample = (f"{rows} of {m} rows of A against {cols} of {n} rows of B, all of K, per step: "
              f"dequantise/upcast + float32 (float64 for s8) matmul, numpy/BLAS")
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": name, "data": "synthetic",
        "config": config_of(work, world),
        "arm": "the reference's CPU path (its correctness oracle) on the host cores, numpy port",
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def algorithmic_bytes_np(name, m, n, k):
    from oracle import opengemm_oracle as ora

    bits = ora.bits_of(name)
    out = {"f32": 4, "s32": 4, "bf16": 2}[ora.FORMATS[name][4]]
    nbytes = (m * k + n * k) * bits // 8 + m * n * out
    if ora.impl_of(name) == "smm":
        nbytes += (m * k + n * k) // ora.sf_block(name)
    return nbytes


def time_launches(torch, fn, steps):
    """Milliseconds for `steps` back-to-back calls of `fn`, by CUDA events on the current stream."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    end.synchronize()
    return start.elapsed_time(end)


class Runner:
    """Operand sets rotated past 2 x L2, the bound kernel, and one-step callables.
    Rank `rank` of `world` owns its rows of B (drawn from its own seed)."""

    def __init__(self, torch, work, device, seed0, world=1, rank=0, max_bytes=24 << 30):
        from opengemm_b200 import capi
        from opengemm_b200.configs import resolve_config
        from opengemm_b200.dtypes import DTYPES
        from opengemm_b200.shard import shard_bounds

        self.torch = torch
        self.name, self.m, self.k = work["name"], work["m"], work["k"]
        n0, n1 = shard_bounds(work["n"], world, rank)
        self.n = n1 - n0
        name, m, n, k = self.name, self.m, self.n, self.k
        self.d = DTYPES[name]
        self.per_set = algorithmic_bytes(name, m, n, k)
        self.copies = int(max(2, min(-(-2 * L2_BYTES // self.per_set), max_bytes // self.per_set)))
        self.sets = []
        for i in range(self.copies):
            ops = make_operands(torch, name, m, n, k, seed0 + i, device, seed_b=(seed0 + i) * 1000 + 7 + rank)
            self.sets.append((ops, torch.empty((m, n), device=device, dtype=self.d.out)))
        # Every operand set here is written once, before any timing, so no kernel of
        # the stream ever produces another's operands: say so, and operand loads of
        # one launch may start while the previous launch drains (stores still wait).
        # Said before the configuration is looked up: the store keeps one per launch mode.
        capi.library(self.d.impl).set_independent_inputs(True)
        self.lib, self.g = capi.bind(name, m, n, k, resolve_config(name, m, n, k))
        self.plan = self.lib.plan(self.g, device.index)
        self.i = 0

    def step(self):
        ops, out = self.sets[self.i % self.copies]
        self.i += 1
        self.lib.launch(self.g, ops.a, ops.b, ops.sfa, ops.sfb, out)

    def parity(self):
        """The first operand set's output against the CPU oracle (sentinel-filled first)."""
        ops, out = self.sets[0]
        out.view(self.torch.uint8).fill_(0x7F)
        self.lib.launch(self.g, ops.a, ops.b, ops.sfa, ops.sfb, out)
        self.torch.cuda.synchronize()
        return sampled_oracle_check(self.torch, self.name, self.k, ops, out)

    def rate(self, us, unit):
        return (self.per_set / us / 1e3) if unit == "GB/s" else (2.0 * self.m * self.n * self.k / us / 1e6)

    def limiter(self):
        """What bounds this shape's per-GPU rate, read off the tile plan."""
        p = self.plan
        slots = SM_COUNT // p["cta_group"]
        waves = p["tiles"] / slots
        if p["tiles"] < slots:
            return f"SM coverage: {p['tiles'] * p['cta_group']} of {SM_COUNT} SMs hold a tile"
        return (f"wave quantisation: {p['tiles']} tiles of {p['tile_m']}x{p['tile_n']} on {slots} "
                f"{'pairs' if p['cta_group'] == 2 else 'CTAs'} = {waves:.2f} waves")


def best_us(torch, fn, steps, repeats=3):
    return min(time_launches(torch, fn, steps) for _ in range(repeats)) * 1e3 / steps


def side_configs(torch, device, skip):
    """The other configurations, measured briefly for the record (not the headline)."""
    results = {}
    for key, steps in (("c1", 100), ("c2", 50), ("c2m", 50), ("c3", 10), ("c4", 6), ("c5", 50)):
        if key == skip:
            continue
        work = WORKLOADS[key]
        try:
            r = Runner(torch, work, device, seed0=50, max_bytes=8 << 30)
            parity = r.parity()
            for _ in range(3):
                r.step()
            torch.cuda.synchronize()
            us = best_us(torch, r.step, steps)
            unit, _ = unit_of(work)
            results[key] = {"dtype": work["name"], "mnk": [r.m, r.n, r.k], "us": round(us, 2),
                            "tflops": round(2.0 * r.m * r.n * r.k / us / 1e6, 1),
                            "gbs": round(r.per_set / us / 1e3, 1), "tile": r.plan, "parity_ok": parity["ok"],
                            "parity_max_rel": parity["max_rel"]}
            if key == "c5":
                # Consecutive launches overlap (each starts loading while its predecessor
                # drains); with the operands declared dependent again every launch waits
                # for the previous one to finish: the single-launch figure.
                # That is the library's default mode, for which the store may hold another plan.
                from opengemm_b200 import capi
                from opengemm_b200.configs import resolve_config
                r.lib.set_independent_inputs(False)
                overlapping = r.g
                r.lib, r.g = capi.bind(r.name, r.m, r.n, r.k, resolve_config(r.name, r.m, r.n, r.k, dependent=True))
                serial = best_us(torch, r.step, steps)
                serial_plan = r.lib.plan(r.g)
                r.g = overlapping
                r.lib.set_independent_inputs(True)
                results[key].update({"us_is": "consecutive launches overlapping", "us_serialised": round(serial, 2),
                                     "gbs_serialised": round(r.per_set / serial / 1e3, 1),
                                     "serialised_tile": f"{serial_plan['tile_m']}x{serial_plan['tile_n']} on {serial_plan['grid']} CTAs"})
            del r
            torch.cuda.empty_cache()
        except Exception as exc:  # a side measurement must never cost the headline
            results[key] = {"error": str(exc)[:160]}
    # The quantisation kernel upstream of the block-scaled GEMMs: bf16 values in,
    # packed nvfp4 + blocked ue4m3 scales out, on c4's B operand shape.
    try:
        import opengemm_b200 as og

        rows, k = 28672, 8192
        xs = [torch.randn((rows, k), device=device).to(torch.bfloat16) for _ in range(2)]
        state = {"i": 0}

        def quantize_step():
            state["i"] += 1
            og.quantize_blocked(xs[state["i"] % 2], "nvfp4")

        for _ in range(3):
            quantize_step()
        torch.cuda.synchronize()
        us = best_us(torch, quantize_step, 10)
        nbytes = rows * k * 2 + rows * k // 2 + rows * k // 16
        results["quantize_nvfp4_28672x8192"] = {"us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1),
                                                "algorithmic_bytes": nbytes}
        del xs
        torch.cuda.empty_cache()
    except Exception as exc:
        results["quantize_nvfp4_28672x8192"] = {"error": str(exc)[:160]}
    # The fp8 product with C rounded to bfloat16 on the way out (an output
    # variant of this build; the reference writes float32 only).
    try:
        from opengemm_b200 import capi
        from opengemm_b200.configs import resolve_config

        work = WORKLOADS["c2"]
        name, m, n, k = work["name"], work["m"], work["n"], work["k"]
        r = Runner(torch, work, device, seed0=70, max_bytes=2 << 30)
        lib, g = capi.bind(name + ".bf16", m, n, k, resolve_config(name, m, n, k))
        outs = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in r.sets]
        state = {"i": 0}

        def bf16_step():
            i = state["i"] % r.copies
            state["i"] += 1
            ops, _ = r.sets[i]
            lib.launch(g, ops.a, ops.b, None, None, outs[i])

        for _ in range(3):
            bf16_step()
        torch.cuda.synchronize()
        us = best_us(torch, bf16_step, 50)
        results["c2_bf16_output"] = {"dtype": name + ".bf16", "mnk": [m, n, k], "us": round(us, 2),
                                     "tflops": round(2.0 * m * n * k / us / 1e6, 1)}
        del r, outs
        torch.cuda.empty_cache()
    except Exception as exc:
        results["c2_bf16_output"] = {"error": str(exc)[:160]}
    return results


def sharded_configs(torch, dist, device, world, rank, skip, shard_counts):
    """The N-sharded configurations, strong-scaled: for each, this rank's shard
    of the `g`-way split timed on every rank at once (max over ranks), the
    whole shape on one GPU beside it, and the per-GPU efficiency between them.
    With one rank, `shard_counts` names the splits whose first shard to time."""
    results = {}
    for key in SHARDED:
        if key == skip:
            continue
        work = WORKLOADS[key]
        unit, _ = unit_of(work)
        steps = {"c3": 10, "c4": 6, "c5": 50}[key]
        try:
            full = Runner(torch, work, device, seed0=90, max_bytes=4 << 30)
            for _ in range(3):
                full.step()
            torch.cuda.synchronize()
            full_us = best_us(torch, full.step, steps)
            full_rate = full.rate(full_us, unit)
            entry = {"dtype": work["name"], "mnk": [full.m, full.n, full.k], "unit": unit,
                     "one_gpu": {"us": round(full_us, 2), "rate": round(full_rate, 1), "limiter": full.limiter()}}
            del full
            torch.cuda.empty_cache()
            for g in shard_counts:
                r = Runner(torch, work, device, seed0=90, world=g, rank=rank if world > 1 else 0, max_bytes=4 << 30)
                parity = r.parity()
                for _ in range(3):
                    r.step()
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                    torch.cuda.synchronize()
                us = best_us(torch, r.step, max(steps, 20))
                if world > 1:
                    t = torch.tensor([us], device=device)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    us = float(t.item())
                rate = r.rate(us, unit)
                entry[f"shard_of_{g}"] = {
                    "mnk": [r.m, r.n, r.k], "us": round(us, 2), "per_gpu_rate": round(rate, 1),
                    "efficiency_vs_one_gpu": round(rate / full_rate, 3), "tile": r.plan, "limiter": r.limiter(),
                    "parity_ok": parity["ok"], "timed_on": f"{world} GPU(s) at once" if world > 1 else "one GPU, first shard",
                }
                del r
                torch.cuda.empty_cache()
            results[key] = entry
        except Exception as exc:
            if world > 1:  # the other ranks are inside the same collectives: fail loudly, not silently apart
                raise
            results[key] = {"error": str(exc)[:200]}
    return results


def library_baseline(torch, r, steps):
    """cuBLAS / cuBLASLt on the first operand set, where torch exposes a kernel for the format."""
    ops, _ = r.sets[0]
    a, b, sfa, sfb = ops.a, ops.b, ops.sfa, ops.sfb
    name = r.name
    one = torch.ones((), device=a.device)
    if name == "bf16":
        f = lambda: torch.mm(a, b.t())
    elif name == "s8":
        f = lambda: torch._int_mm(a, b.t())
    elif name in ("e4m3", "e4m3xe5m2"):
        f = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.float32)
    elif name == "nvfp4":
        f = lambda: torch._scaled_mm(a, b.t(), sfa, sfb, out_dtype=torch.bfloat16)
    else:
        return None
    for _ in range(3):
        f()
    torch.cuda.synchronize()
    return time_launches(torch, f, steps) * 1e3 / steps


def reference_kernel_leg(torch, r, unit):
    """The reference's own sm_100a kernel on the same operand rotation,
    timed in windows alternating with this library's: a side measurement,
    present only when the reference's libraries were built beside the oracle
    (oracle/build_reference_kernels.py).  Never the `--impl reference` arm."""
    from opengemm_b200 import compare

    found = compare.reference_libraries(ROOT / "oracle" / "_ref")
    if found is None:
        return {"unavailable": "the reference's kernel libraries are not built under oracle/_ref"}
    sets = [(ops.a, ops.b, ops.sfa, ops.sfb, out) for ops, out in r.sets]
    result = compare.interleaved(found, r.name, r.m, r.n, r.k, sets, ours=(r.lib, r.g), windows=8, window_ms=60.0)
    if "ref_us" in result:
        result["ref_rate"] = round(r.rate(result["ref_us"], unit), 1)
        result["ours_rate"] = round(r.rate(result["ours_us"], unit), 1)
    return result


def bind_memory_near(device_index):
    """Prefer host memory on the NUMA node of GPU `device_index` for the pages
    this process touches next (the pinned staging buffers), so each rank's
    copies cross its own socket's PCIe root.  Returns a note for the JSON line
    and a callable that puts the thread's CPU affinity and memory policy back."""
    before = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    libc = ctypes.CDLL(None, use_errno=True)
    SYS_set_mempolicy = 238  # x86-64

    def restore():
        try:
            libc.syscall(SYS_set_mempolicy, 0, None, ctypes.c_ulong(0))  # MPOL_DEFAULT
            if before is not None:
                os.sched_setaffinity(0, before)
        except Exception:
            pass

    return _bind_memory_near(device_index, libc, SYS_set_mempolicy), restore


def _bind_memory_near(device_index, libc, SYS_set_mempolicy):
    try:
        import torch

        props = torch.cuda.get_device_properties(device_index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text())
        if node < 0:
            # No placement hint for this GPU: spread the staging pages over every node
            # the process may use, so that several ranks do not all lean on one node's memory.
            online = Path("/sys/devices/system/node/online").read_text().strip()
            nodes = set()
            for part in online.split(","):
                lo, _, hi = part.partition("-")
                nodes.update(range(int(lo), int(hi or lo) + 1))
            if len(nodes) < 2:
                return f"GPU {bus} reports no NUMA node; one node online"
            mask = ctypes.c_ulong(sum(1 << n for n in nodes if n < 64))
            MPOL_INTERLEAVE = 3
            if libc.syscall(SYS_set_mempolicy, MPOL_INTERLEAVE, ctypes.byref(mask), ctypes.c_ulong(64)) != 0:
                return f"GPU {bus} reports no NUMA node; set_mempolicy(interleave) refused: errno {ctypes.get_errno()}"
            return f"GPU {bus} reports no NUMA node; host pages interleaved over nodes {online}"
        mask = ctypes.c_ulong(1 << node)
        MPOL_PREFERRED = 1
        if libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, ctypes.byref(mask), ctypes.c_ulong(64)) != 0:
            return f"set_mempolicy(node {node}) refused: errno {ctypes.get_errno()}"
        cpus = Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip()
        allowed = os.sched_getaffinity(0)
        wanted = set()
        for part in cpus.split(","):
            lo, _, hi = part.partition("-")
            wanted.update(range(int(lo), int(hi or lo) + 1))
        if wanted & allowed:
            os.sched_setaffinity(0, wanted & allowed)
            return f"host pages preferred on NUMA node {node} (GPU {bus}); thread on its CPUs"
        return f"host pages preferred on NUMA node {node} (GPU {bus}); its CPUs are outside this process's affinity"
    except Exception as exc:
        return f"not bound: {str(exc)[:80]}"


def run_ours(args):
    import torch
    import torch.distributed as dist

    import opengemm_b200 as og

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    work = WORKLOADS[args.workload]
    name, m, n_full, k = work["name"], work["m"], work["n"], work["k"]
    r = Runner(torch, work, device, seed0=1000, world=world, rank=rank)
    n = r.n

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # Parity gate: untimed, before the warm-up; every rank checks its own shard.
    parity = r.parity()
    all_ok = max_over_ranks(0.0 if parity["ok"] else 1.0) == 0.0
    if not all_ok:
        if not parity["ok"]:
            print(json.dumps({"parity": parity, "rank": rank, "error": "output outside tolerance; nothing timed"}),
                  file=sys.stderr, flush=True)
        if world > 1:
            dist.destroy_process_group()
        raise SystemExit(3)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        r.step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    t_begin = time.time()
    ms = time_launches(torch, r.step, args.steps)
    barrier()
    ms = max_over_ranks(ms)
    t_end = time.time()
    if ms < 600.0:  # `ms` is the maximum over ranks: every rank takes the same branch
        # the same load a little longer on every rank (no collective inside), so the
        # 100 ms clock sampler sees it; the timed region above is what is reported
        while time.time() - t_begin < 0.6:
            time_launches(torch, r.step, max(args.steps // 4, 1))
        barrier()
        t_end = time.time()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None

    unit, metric = unit_of(work)
    kernel_us = ms * 1e3 / args.steps
    flops_job = 2.0 * m * n_full * k
    bytes_job = algorithmic_bytes(name, m, n_full, k)
    per_gpu = r.rate(kernel_us, unit)                      # this shard's work over the slowest rank's time
    value = (bytes_job / kernel_us / 1e3) if unit == "GB/s" else (flops_job / kernel_us / 1e6)

    # End to end through the public API, every step fed from pinned host memory:
    # host->device copies of the step's operands (A and its scales whole, this
    # rank's rows of B and of B's scales), gemm(), device->host copy of this
    # rank's columns of C.  Three streams and two sets of buffers let step i+1's
    # upload run under step i's download (the link is full duplex); every step
    # still performs all three, in order, on its own buffers.
    numa_note, restore_host_binding = bind_memory_near(local)
    ops0, _ = r.sets[0]
    dev_tensors = [t for t in (ops0.a, ops0.b, ops0.sfa, ops0.sfb) if t is not None]
    host_in = [t.cpu().pin_memory() for t in dev_tensors]
    lanes = []
    for _ in range(2):
        lanes.append({
            "dev_in": [torch.empty_like(t) for t in dev_tensors],
            "dev_c": torch.empty((m, n), device=device, dtype=r.d.out),
            "host_c": torch.empty((m, n), dtype=r.d.out).pin_memory(),
            "uploaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "downloaded": torch.cuda.Event(),
        })
    up, compute, down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    e2e_steps = max(4, min(args.steps, 40))
    state = {"i": 0}

    def e2e_step():
        lane = lanes[state["i"] % 2]
        state["i"] += 1
        with torch.cuda.stream(up):
            up.wait_event(lane["computed"])  # the lane's previous GEMM has read its operands
            for dst, src in zip(lane["dev_in"], host_in):
                dst.copy_(src, non_blocking=True)
            lane["uploaded"].record(up)
        with torch.cuda.stream(compute):
            compute.wait_event(lane["uploaded"])
            compute.wait_event(lane["downloaded"])  # the lane's previous result has left dev_c
            og.gemm(*lane["dev_in"], out=lane["dev_c"])
            lane["computed"].record(compute)
        with torch.cuda.stream(down):
            down.wait_event(lane["computed"])
            lane["host_c"].copy_(lane["dev_c"], non_blocking=True)
            lane["downloaded"].record(down)

    def e2e_run(steps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        current = torch.cuda.current_stream()
        for s in (up, compute, down):
            s.wait_stream(current)
        start.record(up)
        for _ in range(steps):
            e2e_step()
        current.wait_stream(down)
        current.wait_stream(compute)
        current.wait_stream(up)
        end.record(current)
        end.synchronize()
        return start.elapsed_time(end)

    e2e_run(4)
    barrier()
    e2e_ms = e2e_run(e2e_steps)
    barrier()
    e2e_ms = max_over_ranks(e2e_ms)
    e2e_us = e2e_ms * 1e3 / e2e_steps
    e2e_value = (bytes_job / e2e_us / 1e3) if unit == "GB/s" else (flops_job / e2e_us / 1e6)
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = lanes[0]["host_c"].numel() * lanes[0]["host_c"].element_size()
    # the end-to-end output is the product too: same check on this rank's last lane
    e2e_parity = sampled_oracle_check(torch, name, k, ops0, torch.as_tensor(lanes[(state["i"] - 1) % 2]["host_c"]).to(device))
    del lanes, host_in
    torch.cuda.empty_cache()
    restore_host_binding()

    shard_counts = [world] if world > 1 else [2, 4, 8]
    sharded = None if args.no_side else sharded_configs(torch, dist, device, world, rank, None, shard_counts)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    traffic = NCU_TRAFFIC_BYTES.get((name, m, n, k))
    if unit == "GB/s":
        roofline = {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": per_gpu / peaks["hbm_gbs"], "traffic": traffic,
                    "peak_source": f"{peaks['source']} copy bandwidth", "algorithmic_bytes_per_launch": r.per_set}
    else:
        rate = RATE_VS_BF16[name]
        burst = kernel_us * args.steps < 2e6  # a timed region under two seconds runs at burst clocks
        base = peaks["bf16_burst"] if burst else peaks["bf16_sustained"]
        peak = rate * base
        how = "" if rate == 1.0 else f"{rate:g} x "
        roofline = {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
                    "traffic": traffic,
                    "peak_source": f"{how}{peaks['source']} bf16 {'burst' if burst else 'sustained'} ({base} TFLOP/s)"
                                   + ("" if rate == 1.0 else "; this format's own peak is not measured on the pool"),
                    "frac_of_nominal": per_gpu / (rate * NOMINAL_BF16_TFLOPS),
                    "algorithmic_flops_per_launch": 2.0 * m * n * k,
                    "per": "GPU: this rank's shard over the slowest rank's time per launch"}
    try:
        lib_us = library_baseline(torch, r, args.steps)
        roofline["cublas_same_shape"] = None if lib_us is None else r.rate(lib_us, unit)
    except Exception as exc:
        roofline["cublas_same_shape"] = None
        roofline["cublas_note"] = str(exc)[:100]
    if args.no_side or world > 1:
        roofline["reference_kernel_same_shape"] = {
            "unavailable": "side measurements were switched off (--no-side)" if args.no_side
            else "a one-GPU side measurement: not taken under a multi-rank launch"}
    else:
        try:
            roofline["reference_kernel_same_shape"] = reference_kernel_leg(torch, r, unit)
        except Exception as exc:
            roofline["reference_kernel_same_shape"] = {"unavailable": str(exc)[:160]}

    cpu = None
    if world == 1:
        seconds, rows, cols, _ = cpu_sample(name, m, n, k, budget_s=10.0)
        cpu_value = (algorithmic_bytes_np(name, rows, cols, k) / seconds / 1e9) if unit == "GB/s" else (
            2.0 * rows * cols * k / seconds / 1e12)
        cpu = {"value": cpu_value, "unit": unit, "cores": use_all_host_threads(), "kind": "port",
               "sample": f"{rows} of {m} rows of A against {cols} of {n} rows of B, all of K, once ({seconds:.2f} s): "
                         f"dequantise/upcast + float32 (float64 for s8) matmul, numpy/BLAS"}
    others = side_configs(torch, device, args.workload) if (world == 1 and not args.no_side) else None

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": name, "data": "synthetic",
        "config": config_of(work, world),
        "kernel": {
            "shard_mnk": [m, n, k], "tile": r.plan, "limiter": r.limiter(),
            "rotation": f"{r.copies} operand/output sets ({r.copies * r.per_set >> 20} MiB > 2 x L2)",
            "launch": "programmatic dependent launch; operands declared independent of earlier kernels "
                      "(og_b200_set_independent_inputs), output stores wait for the previous grid",
        },
        "parity": parity,
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps, "parity_ok": e2e_parity["ok"],
                "bytes_are": "per rank", "host_memory": numa_note},
        "gpu_launches": args.steps * world, "clocks": clocks,
    }
    if sharded is not None:
        line["sharded_configs"] = sharded
    if others is not None:
        line["other_configs"] = others
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default=HEADLINE,
                        help="which baseline configuration to run (default: c4, the largest single-GPU one)")
    parser.add_argument("--no-side", action="store_true", help="skip the brief measurements of the other configurations")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
