"""The CUDA quantisation kernel (og_b200_quantize, through `og.quantize` and
`og.quantize_blocked` on CUDA tensors) against the numpy oracle of the
reference's quantize + to_blocked.  Byte work: every output byte must match."""

import numpy as np
import pytest
import torch

import opengemm_b200 as og
from oracle import opengemm_oracle as ora

pytestmark = pytest.mark.gpu


def _inputs(kind, rows, k, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == "randn":
        x = torch.randn((rows, k), generator=g) * 3
    elif kind == "uniform":
        x = torch.rand((rows, k), generator=g) * 2 - 1
    elif kind == "wide":  # magnitudes over many binades, exact ties, zeros and a zero block
        x = torch.randn((rows, k), generator=g) * torch.pow(2.0, torch.randint(-12, 12, (rows, 1), generator=g).float())
        x[:, ::7] = 0
        x[0, :64] = 0
        x[1, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("name", ["nvfp4", "mxfp8", "mxfp4"])
@pytest.mark.parametrize("kind", ["randn", "uniform", "wide"])
@pytest.mark.parametrize("shape", [(77, 128), (300, 768), (1024, 4096), (129, 96)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_quantize_kernel_is_bit_exact(name, kind, shape):
    rows, k = shape
    if k % (16 if name == "nvfp4" else 32):
        pytest.skip("K is not a multiple of the scale block")
    x = _inputs(kind, rows, k, seed=rows + k)
    want_packed, want_scales = ora.quantize(ora.bf16_to_f32(x.view(torch.int16).numpy().view(np.uint16)), name)
    want_blocked = ora.to_blocked(want_scales)

    packed, scales = og.quantize(x.cuda(), name)
    torch.cuda.synchronize()
    assert packed.dtype is og.DTYPES[name].a and scales.dtype is og.DTYPES[name].sf
    assert np.array_equal(scales.view(torch.uint8).cpu().numpy(), want_scales)
    assert np.array_equal(packed.view(torch.uint8).cpu().numpy(), want_packed.view(np.uint8).reshape(rows, -1))

    packed2, blocked = og.quantize_blocked(x.cuda(), name)
    torch.cuda.synchronize()
    assert np.array_equal(packed2.view(torch.uint8).cpu().numpy(), want_packed.view(np.uint8).reshape(rows, -1))
    assert np.array_equal(blocked.view(torch.uint8).cpu().numpy(), want_blocked)


def test_quantize_kernel_takes_float32_and_feeds_gemm():
    """float32 input quantises like its own values, and the kernel's outputs
    drive a block-scaled GEMM to the oracle's product."""
    from tests.gemm_util import assert_parity

    m, n, k = 192, 320, 512
    g = torch.Generator().manual_seed(3)
    a32 = torch.randn((m, k), generator=g)
    b32 = torch.randn((n, k), generator=g)
    qa, sfa = og.quantize_blocked(a32.cuda(), "nvfp4")
    qb, sfb = og.quantize_blocked(b32.cuda(), "nvfp4")
    want_a, want_sa = ora.quantize(a32.numpy(), "nvfp4")
    assert np.array_equal(qa.view(torch.uint8).cpu().numpy(), want_a)
    out = og.gemm(qa, qb, sfa, sfb)
    torch.cuda.synchronize()
    want_b, want_sb = ora.quantize(b32.numpy(), "nvfp4")
    case = {"name": "nvfp4", "m": m, "n": n, "k": k, "a": want_a, "b": want_b, "sfa_raw": want_sa, "sfb_raw": want_sb}
    assert_parity(case, out.view(torch.int16).cpu().numpy().view(np.uint16))
