"""Helpers shared by the GPU parity tests: move raw operand bytes to the
device, call the library through its C ABI, and bring the result back."""

import numpy as np
import torch

from opengemm_b200 import capi
from opengemm_b200.configs import heuristic_config
from opengemm_b200.dtypes import DTYPES
from oracle import opengemm_oracle as ora

NP_OUT = {torch.float32: np.float32, torch.int32: np.int32, torch.bfloat16: np.uint16}


def to_device(raw, dtype):
    """A numpy array of storage bytes as a CUDA tensor of `dtype` with the same bytes."""
    t = torch.from_numpy(np.ascontiguousarray(raw))
    if t.dtype == torch.uint16:
        t = t.view(torch.int16)
    return t.cuda().view(dtype)


def make_case(name, m, n, k, seed=0):
    """Seeded operands in the reference's test distribution (bench.py:78-97):
    uniform [-1, 1) floats, full-range integers; returns raw numpy storage."""
    rng = np.random.default_rng(seed)
    impl, ea, eb, bits, out, sf = ora.FORMATS[name]
    case = {"name": name, "m": m, "n": n, "k": k}
    if out == "s32":
        lo, hi = (-127, 128) if name == "s8" else (0, 256)
        case["a"] = rng.integers(lo, hi, (m, k)).astype(np.int8 if name == "s8" else np.uint8)
        case["b"] = rng.integers(lo, hi, (n, k)).astype(np.int8 if name == "s8" else np.uint8)
        return case
    a = (rng.random((m, k), dtype=np.float32) * 2 - 1).astype(np.float32)
    b = (rng.random((n, k), dtype=np.float32) * 2 - 1).astype(np.float32)
    if impl == "smm":
        a = ora.bf16_to_f32(ora.f32_to_bf16(a))
        b = ora.bf16_to_f32(ora.f32_to_bf16(b))
        case["a"], case["sfa_raw"] = ora.quantize(a, name)
        case["b"], case["sfb_raw"] = ora.quantize(b, name)
        case["sfa"] = ora.to_blocked(case["sfa_raw"])
        case["sfb"] = ora.to_blocked(case["sfb_raw"])
        return case

    def store(x, elem):
        if elem == "bf16":
            return ora.f32_to_bf16(x)
        if elem == "f16":
            return x.astype(np.float16).view(np.uint16)
        if elem == "tf32":
            return ora.round_tf32(x)
        if elem == "e4m3":
            return ora.f32_to_e4m3(x)
        if elem == "e5m2":
            return ora.f32_to_e5m2(x)
        return ora.pack(x, elem)

    case["a"], case["b"] = store(a, ea), store(b, eb)
    return case


def golden_case(z, name, m, n, k):
    tag = f"{m}x{n}x{k}"
    case = {"name": name, "m": m, "n": n, "k": k, "a": z[f"{tag}.a"], "b": z[f"{tag}.b"], "c": z[f"{tag}.c"]}
    if ora.impl_of(name) == "smm":
        for key in ("sfa", "sfb", "sfa_raw", "sfb_raw"):
            case[key] = z[f"{tag}.{key}"]
    return case


def oracle_of(case):
    return ora.reference(case["name"], case["a"], case["b"], case.get("sfa_raw"), case.get("sfb_raw"))


def run_library(case, config=None, checked=True):
    """Call og_<impl>_bind + launch for this case; returns the output as numpy
    (float32 / int32 / bf16 bits) after a synchronize."""
    name, m, n, k = case["name"], case["m"], case["n"], case["k"]
    d = DTYPES[name]
    config = config or heuristic_config(name, m, n, k)
    lib, g = capi.bind(name, m, n, k, config)
    a, b = to_device(case["a"], d.a), to_device(case["b"], d.b)
    sfa = to_device(case["sfa"], d.sf) if d.impl == "smm" else None
    sfb = to_device(case["sfb"], d.sf) if d.impl == "smm" else None
    out = torch.empty((m, n), device="cuda", dtype=d.out)
    out.view(torch.uint8).fill_(0x7F)  # sentinel: 0x7f7f7f7f is a huge float / int, 0x7f7f a huge bf16
    if checked:
        lib.set_wait_limit_ms(1000)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        lib.launch_checked(g, a, b, sfa, sfb, out, status)
        torch.cuda.synchronize()
        code = int(status.item())
        assert code == 0, f"device wait gave up: site {code & 0xFF} in CTA {code >> 8} ({lib.plan(g)})"
    else:
        lib.launch(g, a, b, sfa, sfb, out)
        torch.cuda.synchronize()
    if d.out is torch.bfloat16:
        return out.view(torch.int16).cpu().numpy().view(np.uint16)
    return out.cpu().numpy()


def assert_parity(case, got, want=None):
    """Both acceptance rules: the reference's assert_close tolerances and the
    stricter per-format bound of this build (bit-exact for integers)."""
    want = oracle_of(case) if want is None else want
    name, k = case["name"], case["k"]
    ok, worst = ora.check_close(name, k, got, want)
    assert ok, f"{name} {case['m']}x{case['n']}x{k}: outside the reference tolerance by {worst}"
    ok, figure = ora.check_north_star(name, got, want)
    assert ok, f"{name} {case['m']}x{case['n']}x{k}: outside the strict bound ({figure})"
