#!/usr/bin/env python3
"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference checkout is available (it is pure Python on this
path and runs on a CPU):

    python tests/golden/make_golden.py --reference /path/to/OpenGEMM

It imports the reference's own `opengemm.python.bench` / `.quant`, builds its
seeded inputs on the CPU generator (`bench.make_inputs(..., device="cpu")`,
bench.py:78-97), evaluates its oracle (`bench.reference`, bench.py:125-144)
and stores inputs and outputs as raw bytes in `gemm_<dtype>.npz`, the
outputs of the packing / quantising helpers in `quant.npz`, and the distinct
knob sets of its shipped configurations in `reference_config_knobs.json`.  The fixtures
are what pins this repository's oracle to the reference; nothing at test or
benchmark time reads the reference checkout.
"""

import argparse
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SHAPES = [(77, 33, 128), (64, 48, 256), (130, 72, 384)]


def raw(t):
    """A torch tensor's storage bytes as a numpy array of a plain dtype."""
    import torch

    if t is None:
        return np.zeros(0, dtype=np.uint8)
    t = t.contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype in (torch.float32, torch.int32, torch.int8, torch.uint8):
        return t.numpy().copy()
    return t.view(torch.uint8).numpy().copy()  # fp8 / fp4x2 / e8m0


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", required=True, help="a checkout of aramesh10/OpenGEMM (its Python is imported on the CPU)")
    args = parser.parse_args()
    sys.path.insert(0, args.reference)

    import torch
    from opengemm.python import bench, quant
    from opengemm.python.dtypes import DTYPES

    torch.set_num_threads(1)  # a fixed summation order for the float32 products
    for name in DTYPES:
        store = {}
        for m, n, k in SHAPES:
            entry = bench.make_inputs(m, n, k, name, seed=0, device="cpu")
            ref = bench.reference(entry, name)
            tag = f"{m}x{n}x{k}"
            store[f"{tag}.a"] = raw(entry.a)
            store[f"{tag}.b"] = raw(entry.b)
            store[f"{tag}.sfa"] = raw(entry.sfa)
            store[f"{tag}.sfb"] = raw(entry.sfb)
            store[f"{tag}.sfa_raw"] = raw(entry.sfa_raw)
            store[f"{tag}.sfb_raw"] = raw(entry.sfb_raw)
            store[f"{tag}.c"] = raw(ref)
            rtol, atol = bench.tolerance(name, k)
            store[f"{tag}.tol"] = np.asarray([rtol, atol], dtype=np.float64)
        np.savez_compressed(HERE / f"gemm_{name}.npz", **store)
        print("wrote", f"gemm_{name}.npz")

    g = torch.Generator().manual_seed(1)
    x = torch.randn((40, 256), generator=g) * 3
    store = {"x": x.numpy().copy()}
    for elem in ("e3m2", "e2m3", "e2m1"):
        packed = quant.pack(x, elem)
        store[f"pack.{elem}"] = raw(packed)
        store[f"unpack.{elem}"] = quant.unpack(packed, elem, 256).numpy().copy()
        store[f"values.{elem}"] = quant._values(elem, "cpu").numpy().copy()
    store["round_tf32"] = quant.round_tf32(x.clone()).numpy().copy()
    for name in ("nvfp4", "mxfp8", "mxfp4"):
        for tag, src in (("randn", x), ("rand", torch.rand((40, 256), generator=g) * 2 - 1)):
            packed, scales = quant.quantize(src.to(torch.bfloat16), name)
            store[f"quantize.{name}.{tag}.in"] = raw(src.to(torch.bfloat16))
            store[f"quantize.{name}.{tag}.packed"] = raw(packed)
            store[f"quantize.{name}.{tag}.scales"] = raw(scales)
            store[f"quantize.{name}.{tag}.blocked"] = raw(quant.to_blocked(scales))
    odd = torch.arange(200 * 7, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(200, 7)
    store["to_blocked.in"] = raw(odd)
    store["to_blocked.out"] = raw(quant.to_blocked(odd))
    np.savez_compressed(HERE / "quant.npz", **store)
    print("wrote quant.npz")

    # Every distinct (dtype, knob set) of the reference's shipped configs.json
    # files, with one shape it is stored for: bind() must accept all of them.
    import json

    from opengemm.python import capi, configs

    knob_sets = {}
    for impl in ("mm", "smm"):
        seen = {}
        for (dtype, m, n, k), cfg in configs.load_configs(impl).items():
            knobs = {key: int(cfg[key]) for key in capi.KERNEL_KEYS[impl] + capi.LAUNCH_KEYS[impl]}
            sig = (dtype,) + tuple(sorted(knobs.items()))
            seen.setdefault(sig, {"dtype": dtype, "m": m, "n": n, "k": k, "config": knobs})
        knob_sets[impl] = list(seen.values())
    (HERE / "reference_config_knobs.json").write_text(json.dumps(knob_sets, separators=(",", ":")))
    print("wrote reference_config_knobs.json")


if __name__ == "__main__":
    main()
