"""Host-side logic that needs no GPU: format naming, operand checks, the
configuration store, the torch packing/quantising helpers against fixtures
made by the reference, and the N-shard bookkeeping."""

import json
import os

import numpy as np
import pytest
import torch

import opengemm_b200 as og
from opengemm_b200 import api, configs, quant, shard
from opengemm_b200.dtypes import DTYPES, dtype_name, extent, k_of, sf_block
from oracle import opengemm_oracle as ora


def test_public_names_are_the_references():
    assert set(og.__all__) == {"gemm", "prebuild", "emit_kernel", "run_kernel", "dtype_name", "DTYPES",
                               "quantize", "to_blocked", "pack", "unpack"}
    assert list(DTYPES) == list(ora.FORMATS)
    impl, a, b, bits, out, sf = DTYPES["nvfp4"]
    assert (impl, bits, out, sf) == ("smm", 4, torch.bfloat16, torch.float8_e4m3fn)


def test_dtype_name_rules():
    bf = torch.zeros((2, 8), dtype=torch.bfloat16)
    u8 = torch.zeros((2, 8), dtype=torch.uint8)
    e4 = torch.zeros((2, 16), dtype=torch.float8_e4m3fn)
    e5 = torch.zeros((2, 16), dtype=torch.float8_e5m2)
    assert dtype_name(bf, bf) == "bf16"
    assert dtype_name(e4, e5) == "e4m3xe5m2"
    assert dtype_name(u8, u8, atype="e2m1") == "e2m1"
    assert dtype_name(atype="e2m1", sftype="ue4m3") == "nvfp4"
    assert dtype_name(atype="e2m1", sftype="ue8m0") == "mxfp4"
    assert dtype_name(e4, e4, torch.zeros(512, dtype=torch.float8_e8m0fnu)) == "mxfp8"
    with pytest.raises(TypeError, match="names no element"):
        dtype_name(u8, u8)
    with pytest.raises(TypeError, match="not a format this build serves"):
        dtype_name(e5, e4)
    with pytest.raises(TypeError, match="without operands"):
        dtype_name()
    d = DTYPES["e3m2"]
    assert extent(d, 128) == 96 and k_of(d, 96) == 128
    assert sf_block(DTYPES["nvfp4"]) == 16 and sf_block(DTYPES["mxfp8"]) == 32


def test_operand_checks_raise_the_references_errors():
    a = torch.zeros((4, 64), dtype=torch.bfloat16)
    with pytest.raises(TypeError, match="a must be a contiguous 2-D CUDA tensor"):
        og.gemm(a, a)
    d = DTYPES["nvfp4"]
    assert api.scale_bytes(d, 8192, 8192) == 8192 * 512 and api.scale_bytes(d, 64, 8192) == 128 * 512
    assert api.scale_bytes(DTYPES["mxfp4"], 57344, 8192) == 57344 * 256
    with pytest.raises(ValueError, match="out must be a contiguous"):
        api.output(DTYPES["bf16"], 4, 4, torch.zeros((4, 5)), torch.device("cpu"))


def test_torch_quant_helpers_match_reference_fixtures(golden_dir):
    z = np.load(golden_dir / "quant.npz")
    x = torch.from_numpy(z["x"])
    for elem in ("e3m2", "e2m3", "e2m1"):
        assert np.array_equal(quant.pack(x, elem).numpy(), z[f"pack.{elem}"])
        assert np.array_equal(quant.unpack(torch.from_numpy(z[f"pack.{elem}"]), elem, 256).numpy(), z[f"unpack.{elem}"])
    assert np.array_equal(quant.round_tf32(x.clone()).numpy(), z["round_tf32"])
    assert np.array_equal(quant.to_blocked(torch.from_numpy(z["to_blocked.in"])).numpy(), z["to_blocked.out"])
    for name in ("nvfp4", "mxfp8", "mxfp4"):
        for tag in ("randn", "rand"):
            src = torch.from_numpy(z[f"quantize.{name}.{tag}.in"].view(np.int16)).view(torch.bfloat16)
            packed, scales = quant.quantize(src, name)
            assert np.array_equal(packed.view(torch.uint8).numpy(), z[f"quantize.{name}.{tag}.packed"])
            assert np.array_equal(scales.view(torch.uint8).numpy(), z[f"quantize.{name}.{tag}.scales"])
            assert np.array_equal(quant.to_blocked(scales).view(torch.uint8).numpy(), z[f"quantize.{name}.{tag}.blocked"])


def test_config_store_round_trip(tmp_path, monkeypatch):
    monkeypatch.setenv("OPENGEMM_CONFIGS", str(tmp_path))
    assert configs.stored_entry("bf16", 96, 96, 96) is None
    cfg = configs.resolve_config("bf16", 96, 96, 96)  # nothing stored: the heuristic answers, for dependent launches by default
    assert cfg == configs.heuristic_config("bf16", 96, 96, 96, dependent=True)
    assert configs.resolve_config("bf16", 96, 96, 96, dependent=False) == configs.heuristic_config("bf16", 96, 96, 96)
    entry = {"dtype": "bf16", "m": 96, "n": 96, "k": 96, "config": dict(cfg, output_n=32)}
    path = configs.write_entry("mm", entry)
    assert path == tmp_path / "tuned_configs.json"
    assert configs.resolve_config("bf16", 96, 96, 96)["output_n"] == 32
    configs.write_entry("mm", {"dtype": "bf16", "m": 96, "n": 96, "k": 96, "config": dict(cfg, output_n=48)})
    configs.write_entry("smm", {"dtype": "nvfp4", "m": 1, "n": 2, "k": 64, "config": None, "unimplementable": "too small"})
    store = json.loads(path.read_text())
    assert store["arch"] == "sm_100" and [e["dtype"] for e in store["entries"]] == ["bf16", "nvfp4"]
    assert configs.resolve_config("bf16", 96, 96, 96)["output_n"] == 48
    with pytest.raises(ValueError, match="cannot be served: too small"):
        configs.resolve_config("nvfp4", 1, 2, 64)
    assert not list(tmp_path.glob("*.tmp"))


def test_a_format_without_an_entry_takes_its_kernel_familys(tmp_path, monkeypatch):
    monkeypatch.setenv("OPENGEMM_CONFIGS", str(tmp_path))
    shape = (96, 200, 160)
    odd = dict(configs.heuristic_config("e4m3", *shape), output_n=80, supergroup=3)
    configs.write_entry("mm", {"dtype": "e4m3", "m": shape[0], "n": shape[1], "k": shape[2], "config": odd})
    for name in ("e5m2", "e2m1", "e4m3xe5m2"):
        assert configs.resolve_config(name, *shape) == odd
    assert configs.resolve_config("bf16", *shape) == configs.heuristic_config("bf16", *shape, dependent=True)  # another kernel
    own = dict(odd, output_n=96)
    configs.write_entry("mm", {"dtype": "e5m2", "m": shape[0], "n": shape[1], "k": shape[2], "config": own})
    assert configs.resolve_config("e5m2", *shape) == own  # its own entry wins


def test_an_entry_may_hold_one_configuration_per_launch_mode(tmp_path, monkeypatch):
    monkeypatch.setenv("OPENGEMM_CONFIGS", str(tmp_path))
    shape = (64, 7168, 8192)
    fat = dict(configs.heuristic_config("mxfp4", *shape), output_n=256)
    wide = dict(fat, output_n=64)
    configs.write_entry("smm", {"dtype": "mxfp4", "m": shape[0], "n": shape[1], "k": shape[2], "config": fat})
    assert configs.resolve_config("mxfp4", *shape, dependent=False) == fat
    # tuned for overlapping launches only, on 28 of 148 SMs: a dependent launch takes the rule's plan instead
    spread = configs.resolve_config("mxfp4", *shape)
    assert configs.planned_ctas(fat, 64, 7168) == 28 and configs.planned_ctas(spread, 64, 7168) >= 100
    full = dict(fat, output_n=32)  # an entry that already covers the GPU serves both modes
    configs.write_entry("smm", {"dtype": "mxfp4", "m": 64, "n": 8192, "k": 4096, "config": full})
    assert configs.resolve_config("mxfp4", 64, 8192, 4096) == full
    configs.write_entry("smm", {"dtype": "mxfp4", "m": shape[0], "n": shape[1], "k": shape[2], "config": fat,
                                "config_dependent": wide})
    assert configs.resolve_config("mxfp4", *shape, dependent=True) == wide
    assert configs.resolve_config("mxfp4", *shape, dependent=False) == fat
    assert configs.resolve_config("mxfp4", *shape) == wide  # the library's default mode is the dependent one
    # the heuristic spreads a dependent decode launch over more CTAs than an independent one
    a, b = configs.heuristic_config("mxfp4", 64, 7000, 8192), configs.heuristic_config("mxfp4", 64, 7000, 8192, dependent=True)
    assert a["output_n"] >= b["output_n"]


def test_config_store_reads_a_file_in_the_references_schema(tmp_path, monkeypatch, golden_dir):
    sets = json.loads((golden_dir / "reference_config_knobs.json").read_text())
    ref_entry = dict(sets["mm"][0])
    ref_entry["config"] = {k: bool(v) if k in ("use_2cta", "use_clc", "swap_ab") else v for k, v in ref_entry["config"].items()}
    (tmp_path / "tuned_configs.json").write_text(json.dumps({"kind": "mm", "arch": "sm_100", "entries": [ref_entry]}))
    monkeypatch.setenv("OPENGEMM_CONFIGS", str(tmp_path))
    got = configs.resolve_config(ref_entry["dtype"], ref_entry["m"], ref_entry["n"], ref_entry["k"])
    assert got == ref_entry["config"]


def test_shard_bounds_cover_n_on_block_boundaries():
    for n in (1024, 3584, 28672, 57344, 8192, 520, 77):
        for world in (1, 2, 4, 8):
            spans = [shard.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(s[0] % 128 == 0 or s[0] == n for s in spans)  # empty trailing shards start at n
    with pytest.raises(ValueError):
        shard.shard_bounds(1024, 4, 4)


def test_shard_of_blocked_scales_is_the_blocked_shard():
    """Cutting the flat blocked buffer on 128-row boundaries equals blocking the cut scales."""
    rng = np.random.default_rng(0)
    n, k, name = 640, 512, "nvfp4"
    raw = rng.integers(1, 120, (n, k // 16)).astype(np.uint8)
    flat = torch.from_numpy(ora.to_blocked(raw))
    for world in (2, 4):
        for rank in range(world):
            n0, n1 = shard.shard_bounds(n, world, rank)
            part = shard.shard_scales(flat, name, n, k, world, rank).numpy()
            assert np.array_equal(part, ora.to_blocked(raw[n0:n1]))


def test_the_shape_suite_lists_the_headline_configurations():
    from opengemm_b200.configs import load_shapes

    shapes = load_shapes()
    assert len(shapes) >= 68 and len(set(shapes)) == len(shapes)
    for shape in [(1024, 1024, 1024), (4096, 4096, 4096), (8192, 8192, 8192), (8192, 28672, 8192), (64, 57344, 8192),
                  (8192, 1024, 8192), (8192, 3584, 8192), (64, 7168, 8192)]:
        assert shape in shapes


def test_heuristic_configurations_follow_the_tile_time_model():
    """Wide pair tiles for long-K compute-bound shapes, single CTAs once the
    output stores dominate, operand swap for small M, the measured corrections
    (fp4 decode, block-scaled tile width, launch-bound shapes); every choice binds."""
    from opengemm_b200 import capi
    from opengemm_b200.configs import heuristic_config, load_shapes, modelled_us

    big = heuristic_config("e4m3", 8192, 8192, 8192)
    assert big["use_2cta"] and big["output_n"] == 256 and not big["swap_ab"]
    assert not heuristic_config("bf16", 8192, 8192, 32)["use_2cta"]
    decode = heuristic_config("mxfp4", 64, 57344, 8192)   # fp4 decode: fat single-CTA tiles, no swap
    assert not decode["swap_ab"] and not decode["use_2cta"] and decode["output_n"] == 256
    assert heuristic_config("e4m3", 16, 8192, 4096)["swap_ab"]   # other small-M shapes ride the N side
    scaled = heuristic_config("nvfp4", 8192, 14336, 8192)       # two accumulators beat one 256-wide tile
    assert scaled["use_2cta"] and scaled["output_n"] == 192
    tiny = heuristic_config("bf16", 128, 128, 128)               # launch-bound: one fat CTA, not four thin ones
    assert not tiny["use_2cta"] and tiny["output_n"] == 128
    # a narrow tile never models faster than the full-width pair tile on a long-K square
    assert modelled_us("bf16", 8192, 8192, 8192, True, 64, False) > modelled_us("bf16", 8192, 8192, 8192, True, 256, False)
    for name in ("bf16", "s8", "e2m3", "nvfp4", "mxfp8", "mxfp4"):
        for m, n, k in load_shapes():
            try:
                capi.bind(name, m, n, k, heuristic_config(name, m, n, k))
            except RuntimeError as exc:  # only K granularity may refuse a suite shape
                assert "multiple" in str(exc), (name, m, n, k, str(exc))


def test_bf16_output_variants_bind_and_stay_out_of_the_reference_tables():
    """The "<format>.bf16" names exist for dense float formats only, run their
    format's tile plan with 2-byte output, and appear neither in DTYPES nor in
    the kernel menu a reference-side tuner walks."""
    import opengemm_b200 as og
    from opengemm_b200 import capi
    from opengemm_b200.configs import heuristic_config
    from opengemm_b200.dtypes import BF16_OUT, DTYPES, base_name, lookup

    assert len(DTYPES) == 14 and sorted(BF16_OUT) == sorted(
        n + ".bf16" for n, d in DTYPES.items() if d.impl == "mm" and d.out is torch.float32)
    assert base_name("e4m3xe5m2.bf16") == "e4m3xe5m2" and base_name("nvfp4") == "nvfp4"
    assert lookup("tf32.bf16").out is torch.bfloat16 and lookup("tf32").out is torch.float32
    for name in BF16_OUT:
        lib, g = capi.bind(name, 512, 768, 1024, heuristic_config(base_name(name), 512, 768, 1024))
        described = lib.describe(g)
        assert described["out_bytes"] == 2 and 14 <= described["variant"] <= 19
    mm = capi.library("mm")
    assert all("." not in row["dtype"] for row in mm.kernels())
    with pytest.raises(TypeError):
        lookup("s8.bf16")
    from opengemm_b200 import emit

    with pytest.raises(ValueError):  # standalone kernels are emitted for the fourteen formats only
        emit.emit("e4m3.bf16", 256, 256, 256, heuristic_config("e4m3", 256, 256, 256), "mm_e4m3_256_256_256")


def test_suite_report_summary_counts_and_geometric_mean():
    from opengemm_b200.benchmark import summarise

    rows = [
        {"dtype": "bf16", "status": "ok", "speedup": 2.0},
        {"dtype": "bf16", "status": "ok", "speedup": 0.5},
        {"dtype": "bf16", "status": "skipped: K too small"},
        {"dtype": "bf16", "status": "INCORRECT: mismatch"},
        {"dtype": "mxfp4", "status": "ok"},  # no library kernel to compare with
    ]
    out = summarise(rows)
    assert out["bf16"] == {"measured": 2, "skipped": 1, "incorrect": 1, "geomean_speedup": 1.0, "below_0.95": 1}
    assert out["mxfp4"]["geomean_speedup"] is None and out["mxfp4"]["measured"] == 1


def test_build_staleness_is_by_content_and_the_cache_follows_the_environment(tmp_path, monkeypatch):
    """The in-tree library is current while its stamp matches the sources'
    content (touching a file changes nothing; another digest does), and the
    cache location and the JIT switch follow the reference's environment
    variables (opengemm/python/build.py:21-24,104-125)."""
    import json
    import os

    from opengemm_b200 import build

    assert not build.stale()
    header = build.CSRC / "raster.h"
    before = header.stat()
    os.utime(header, None)                       # a newer modification time, same content
    try:
        assert not build.stale()
    finally:
        os.utime(header, (before.st_atime, before.st_mtime))
    stamp = build.LIB_DIR / "stamp.json"
    saved = stamp.read_text()
    try:
        stamp.write_text(json.dumps({"sources": "0" * 16}))
        assert build.stale()
    finally:
        stamp.write_text(saved)
    monkeypatch.setenv("OPENGEMM_CACHE", str(tmp_path / "cache"))
    assert build.cache_dir() == tmp_path / "cache"
    monkeypatch.delenv("OPENGEMM_CACHE")
    monkeypatch.setenv("XDG_CACHE_HOME", str(tmp_path / "xdg"))
    assert build.cache_dir() == tmp_path / "xdg" / "opengemm_b200"
    # OPENGEMM_JIT sets the in-tree library aside for the cached one of this exact build
    monkeypatch.setenv("OPENGEMM_JIT", "1")
    expected = build.cache_dir() / build.build_hash() / build.LIB_NAME
    expected.parent.mkdir(parents=True)
    expected.write_bytes(b"placeholder")        # present already: nothing is compiled
    assert build.library_path("mm") == expected
    monkeypatch.setenv("OPENGEMM_LIB_MM", "/somewhere/else.so")
    assert str(build.library_path("mm")) == "/somewhere/else.so"


def test_heuristic_makes_the_tuned_pair_or_single_choice_on_most_shipped_entries():
    """A guard on the rule that serves untuned shapes: against what tuning found,
    per launch mode, over the whole shipped store."""
    for dependent, key in ((False, "config"), (True, "config_dependent")):
        same = total = 0
        for impl in ("mm", "smm"):
            for e in json.loads(configs.config_path(impl).read_text())["entries"]:
                tuned = e.get(key)
                if tuned is None:
                    continue
                ruled = configs.heuristic_config(e["dtype"], e["m"], e["n"], e["k"], dependent=dependent)
                same += bool(ruled["use_2cta"]) == bool(tuned["use_2cta"])
                total += 1
        assert total >= 300 and same >= 0.8 * total, (dependent, same, total)


def test_tuning_one_launch_mode_keeps_the_other_modes_configuration():
    from opengemm_b200 import tune

    fat, wide = {"output_n": 256}, {"output_n": 64}
    first = tune.merged_entry(None, "mxfp4", 64, 7168, 8192, fat, {"us": 5.4}, dependent=False)
    assert first == {"dtype": "mxfp4", "m": 64, "n": 7168, "k": 8192, "config": fat, "measured": {"us": 5.4}}
    both = tune.merged_entry(first, "mxfp4", 64, 7168, 8192, wide, {"us": 10.7}, dependent=True)
    assert both["config"] == fat and both["config_dependent"] == wide and both["measured_dependent"] == {"us": 10.7}
    again = tune.merged_entry(both, "mxfp4", 64, 7168, 8192, dict(fat, supergroup=1), {"us": 5.3}, dependent=False)
    assert again["config"]["supergroup"] == 1 and again["config_dependent"] == wide and again["measured"] == {"us": 5.3}
    alone = tune.merged_entry(None, "mxfp4", 64, 7168, 8192, wide, {"us": 10.7}, dependent=True)
    assert alone["config"] == wide and alone["config_dependent"] == wide  # a store entry always has `config`
