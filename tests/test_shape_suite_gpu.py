"""The whole shape suite at full size, with the configuration gemm() would
pick.  Operands are generated on the GPU; the CPU oracle then recomputes a
sample of output rows and columns (first, last, tile seams, random) from the
matching rows of A and B, which is exact for a product whose entries depend on
one row of each operand.  Each shape takes three of the fourteen formats in
rotation, so every format meets about seventeen shapes."""

import numpy as np
import pytest
import torch

import bench
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
    rows, cols = bench.sample_indices(m, rng), bench.sample_indices(n, rng)
    raw_rows = lambda t, index: bench.raw_rows(torch, t, index)
    sfa = raw_rows(inputs.sfa_raw, rows) if d.impl == "smm" else None
    sfb = raw_rows(inputs.sfb_raw, cols) if d.impl == "smm" else None
    want = ora.reference(name, raw_rows(inputs.a, rows), raw_rows(inputs.b, cols), sfa, sfb)
    picked = out[torch.as_tensor(rows).cuda()][:, torch.as_tensor(cols).cuda()].contiguous()
    got = picked.view(torch.int16).cpu().numpy().view(np.uint16) if d.out is torch.bfloat16 else picked.cpu().numpy()
    ok, worst = ora.check_close(name, k, got, want)
    assert ok, f"{name} {m}x{n}x{k}: outside the reference tolerance by {worst}"
    ok, figure = ora.check_north_star(name, got, want)
    assert ok, f"{name} {m}x{n}x{k}: outside the strict bound ({figure})"
    del inputs, out
    torch.cuda.empty_cache()
