"""The whole shape suite at full size, with the configuration gemm() would
pick.  Operands are generated on the GPU; the CPU oracle then recomputes a
sample of output rows and columns (first, last, tile seams, random) from the
matching rows of A and B, which is exact for a product whose entries depend on
one row of each operand.  Each shape takes three of the fourteen formats in
rotation, so every format meets about seventeen shapes."""

import numpy as np
import pytest
import torch

from opengemm_b200 import capi, configs, harness
from opengemm_b200.dtypes import DTYPES
from oracle import opengemm_oracle as ora

pytestmark = pytest.mark.gpu

NAMES = list(ora.FORMATS)
SHAPES = configs.load_shapes()
CASES = [(NAMES[(3 * i + j) % len(NAMES)], shape) for i, shape in enumerate(SHAPES) for j in range(3)]
# the two large shapes of the reference's own test list (scripts/test.py:23-30), for every format
for _shape in [(2048, 2048, 2048), (1, 8192, 8192)]:
    CASES += [(name, _shape) for name in NAMES if (name, _shape) not in CASES]
SAMPLE = 40


def sample_indices(extent, rng):
    """Up to SAMPLE indices: both ends, both sides of every 128 / 256 seam near
    the ends and the middle, the rest random."""
    seams = [0, extent - 1]
    for at in (128, 192, 256, extent // 2 // 128 * 128, (extent - 1) // 256 * 256):
        seams += [at - 1, at]
    picks = [i for i in dict.fromkeys(seams) if 0 <= i < extent]
    spare = SAMPLE - len(picks)
    if spare > 0 and extent > len(picks):
        picks += list(rng.choice(extent, size=min(spare, extent), replace=False))
    return np.array(sorted(set(int(i) for i in picks))[:SAMPLE])


def raw_rows(t, rows):
    """Selected rows of a device tensor as the storage-typed numpy array the oracle reads."""
    index = torch.from_numpy(rows).to(t.device)
    if t.dtype in (torch.float32, torch.int8, torch.uint8):
        return t[index].cpu().numpy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16)[index].cpu().numpy().view(np.uint16)
    return t.view(torch.uint8)[index].cpu().numpy()  # fp8 codes, packed fp4 pairs


@pytest.mark.parametrize("name,shape", CASES, ids=[f"{n}-{'x'.join(map(str, s))}" for n, s in CASES])
def test_suite_shape_matches_the_oracle_on_sampled_rows_and_columns(name, shape):
    m, n, k = shape
    d = DTYPES[name]
    config = configs.resolve_config(name, m, n, k)
    try:
        lib, g = capi.bind(name, m, n, k, config)
    except RuntimeError as exc:
        pytest.skip(str(exc)[:120])  # K below the multiple this format's tensor maps need
    inputs = harness.make_inputs(m, n, k, name, seed=5)
    out = torch.empty((m, n), device="cuda", dtype=d.out)
    out.view(torch.uint8).fill_(0x7F)
    lib.set_wait_limit_ms(2000)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.launch_checked(g, inputs.a, inputs.b, inputs.sfa, inputs.sfb, out, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device wait gave up: {int(status.item())} ({lib.plan(g)})"

    rng = np.random.default_rng(m * 31 + n * 17 + k)
    rows, cols = sample_indices(m, rng), sample_indices(n, rng)
    sfa = raw_rows(inputs.sfa_raw, rows) if d.impl == "smm" else None
    sfb = raw_rows(inputs.sfb_raw, cols) if d.impl == "smm" else None
    want = ora.reference(name, raw_rows(inputs.a, rows), raw_rows(inputs.b, cols), sfa, sfb)
    picked = out[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].contiguous()
    got = picked.view(torch.int16).cpu().numpy().view(np.uint16) if d.out is torch.bfloat16 else picked.cpu().numpy()
    ok, worst = ora.check_close(name, k, got, want)
    assert ok, f"{name} {m}x{n}x{k}: outside the reference tolerance by {worst}"
    ok, figure = ora.check_north_star(name, got, want)
    assert ok, f"{name} {m}x{n}x{k}: outside the strict bound ({figure})"
    del inputs, out
    torch.cuda.empty_cache()
