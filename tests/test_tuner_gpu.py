"""The autotuner end to end on one small shape: it sweeps tile geometry and,
around the leaders, pipeline depth, the cluster-launch-control scheduler,
rasterisation and the other launch axes; keeps only candidates that reproduce
the reference product; writes the winner in the configs.json schema of the
reference (opengemm/python/configs.py:15-105) into the local store; and
gemm() then resolves that entry."""

import json

import pytest
import torch

import opengemm_b200 as og
from opengemm_b200 import api, capi, configs, tune

def test_refinements_cover_pipeline_depth_scheduler_and_rasterisation():
    base = tune.base_config("bf16", use_2cta=True, output_n=256)
    around = tune.refinements(base, tiles_n=16, fit_stages=6)
    assert {c["stages"] for c in around if c["stages"]} >= {5, 4, 3, 2}
    assert any(c["use_clc"] for c in around) and any(c["walk"] == 1 for c in around) and any(c["walk"] == 3 for c in around)
    assert any(c["split_k"] == 2 for c in around) and any(c["l2_promo"] == 2 for c in around)
    assert tune.simplicity(base) < min(tune.simplicity(c) for c in around if c["supergroup"] == base["supergroup"])


@pytest.mark.gpu
@pytest.mark.parametrize("name,shape", [("e4m3", (512, 768, 1024)), ("mxfp4", (256, 640, 1024))])
def test_tune_writes_a_correct_entry_that_gemm_then_resolves(name, shape, tmp_path, monkeypatch):
    m, n, k = shape
    monkeypatch.setenv("OPENGEMM_CONFIGS", str(tmp_path))
    best = tune.tune(name, m, n, k, window_ms=2.0, final_ms=4.0)
    store = json.loads((tmp_path / configs.TUNED_FILE).read_text())
    assert store["arch"] == "sm_100" and len(store["entries"]) == 1
    entry = store["entries"][0]
    assert (entry["dtype"], entry["m"], entry["n"], entry["k"]) == (name, m, n, k)
    assert entry["config"] == best and entry["measured"]["us"] > 0 and "gpu" in entry["measured"]["env"]
    impl = og.DTYPES[name].impl
    assert set(capi.KERNEL_KEYS[impl]) <= set(best) | {"block_m", "epi_hold", "epi_double"}  # the schema's kernel keys
    assert configs.resolve_config(name, m, n, k, dependent=False) == best
    # the same shape tuned for launches that wait for their predecessor lands beside it
    serial = tune.tune(name, m, n, k, window_ms=2.0, final_ms=4.0, dependent=True)
    entry = json.loads((tmp_path / configs.TUNED_FILE).read_text())["entries"][0]
    assert entry["config"] == best and entry["config_dependent"] == serial and entry["measured_dependent"]["us"] > 0
    assert configs.resolve_config(name, m, n, k) == serial  # the library's default mode
    assert not capi.independent_inputs()  # the tuner put the caller's mode back
    # the stored entry is what a bound GEMM now runs, and it is correct
    from opengemm_b200 import harness

    inputs = harness.make_inputs(m, n, k, name, seed=1)
    api.forget(name)
    out = og.gemm(inputs.a, inputs.b, inputs.sfa, inputs.sfb)
    torch.cuda.synchronize()
    rtol, atol = harness.tolerance(name, k)
    torch.testing.assert_close(out, harness.reference(inputs, name), rtol=rtol, atol=atol)
    api.forget(name)
