"""The C ABI without a GPU: the library loads, exports every declared symbol,
speaks ABI 3, validates like the reference's bind, and plans tiles.  No
compute call is made here."""

import ctypes
import json
import re
from ctypes import byref
from pathlib import Path

import pytest
import torch

from opengemm_b200 import capi
from opengemm_b200.configs import heuristic_config
from opengemm_b200.dtypes import DTYPES

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "opengemm_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"OG_API\s+[\w\s\*]+?\b(og_\w+)\s*\(", text)


def test_every_declared_symbol_is_exported():
    lib = ctypes.CDLL(str(capi.library("mm").path))
    names = declared_symbols()
    assert len(names) >= 15 and len(set(names)) == len(names)
    for name in names:
        assert getattr(lib, name) is not None, name


def test_abi_version_and_struct_size():
    assert ctypes.sizeof(capi.OgGemm) == 108
    for impl in ("mm", "smm"):
        assert capi.library(impl)._abi() == 3


@pytest.mark.parametrize("impl", ["mm", "smm"])
def test_every_menu_row_binds(impl):
    lib = capi.library(impl)
    rows = lib.kernels()
    assert rows and {r["dtype"] for r in rows} == {n for n, d in DTYPES.items() if d.impl == impl}
    for row in rows:
        g = lib.bind(row["dtype"], 512, 512, 512, row)
        plan = lib.plan(g)
        assert plan["stages"] >= 2 and plan["tmem_cols"] <= 512 and plan["smem_bytes"] <= 227 * 1024 - 1024
        assert plan["cta_group"] == (2 if row["use_2cta"] else 1)
        assert plan["tile_n"] % 16 == 0 and plan["tile_n"] <= 256


def test_bind_errors_match_the_reference_contract():
    lib = capi.library("mm")
    g = capi.OgGemm(m=16, n=16, k=64, dtype=b"nope")
    assert lib._bind(byref(g)) == capi.OG_ERR_BIND and "names no element pair" in lib.error()
    g = capi.OgGemm(m=0, n=16, k=64, dtype=b"bf16")
    assert lib._bind(byref(g)) == capi.OG_ERR_BIND and "must be positive" in lib.error()
    g = capi.OgGemm(m=16, n=16, k=12, dtype=b"bf16")
    assert lib._bind(byref(g)) == capi.OG_ERR_BIND
    assert lib.error() == "K = 12 is not a multiple of 8, which the tensor map for bf16 requires"
    g = capi.OgGemm(m=16, n=16, k=192, dtype=b"e2m1")  # sub-byte dense formats need whole 128-value groups
    assert lib._bind(byref(g)) == capi.OG_ERR_BIND and "multiple of 128" in lib.error()
    g = capi.OgGemm(m=16, n=16, k=64, dtype=b"nvfp4")  # a block-scaled name through the dense entry point
    assert lib._bind(byref(g)) == capi.OG_ERR_BIND and "og_smm_bind" in lib.error()
    smm = capi.library("smm")
    g = capi.OgGemm(m=16, n=16, k=48, dtype=b"mxfp8")
    assert smm._bind(byref(g)) == capi.OG_ERR_BIND and "multiple of 32" in smm.error()


def test_launch_before_bind_is_refused():
    lib = capi.library("mm")
    g = capi.OgGemm(m=128, n=128, k=128, dtype=b"bf16", output_n=128, row=-1)
    status = lib._launch(byref(g), 1, 1, 0, 0, 1, 0, 0)  # never reaches the GPU: row does not match
    assert status == capi.OG_ERR_LAUNCH and "bind it first" in lib.error()


def test_split_k_is_clamped_like_the_reference():
    lib = capi.library("mm")
    g = lib.bind("bf16", 64, 64, 512, dict(heuristic_config("bf16", 64, 64, 512), split_k=64))
    assert g.split_k == 4  # never more than ceil(K / 128)
    g = lib.bind("bf16", 64, 64, 512, dict(heuristic_config("bf16", 64, 64, 512), split_k=8, epi_double=1))
    assert g.split_k == 1


def test_all_shipped_reference_knob_sets_bind(golden_dir):
    """Every distinct knob set of the reference's own configs.json files binds
    (keys with no native counterpart are mapped, not refused)."""
    sets = json.loads((golden_dir / "reference_config_knobs.json").read_text())
    for impl in ("mm", "smm"):
        lib = capi.library(impl)
        assert len(sets[impl]) > 50
        for e in sets[impl]:
            g = lib.bind(e["dtype"], e["m"], e["n"], e["k"], e["config"])
            assert lib.plan(g)["tiles"] >= 1


def test_every_shipped_configuration_binds():
    """Both configurations of every entry of the shipped store (one per launch
    mode where tuning found two) bind, and carry the measurement they came from."""
    from opengemm_b200 import configs

    total = second = 0
    for impl in ("mm", "smm"):
        lib = capi.library(impl)
        for e in json.loads(configs.config_path(impl).read_text())["entries"]:
            total += 1
            assert lib.plan(lib.bind(e["dtype"], e["m"], e["n"], e["k"], e["config"]))["tiles"] >= 1
            assert e["measured"]["us"] > 0
            if e.get("config_dependent") is not None:
                second += 1
                assert e["config_dependent"] != e["config"] and e["measured_dependent"]["us"] > 0
                assert lib.plan(lib.bind(e["dtype"], e["m"], e["n"], e["k"], e["config_dependent"]))["tiles"] >= 1
    assert total >= 400 and second >= 100


def test_plan_of_the_baseline_configurations():
    for name, m, n, k in [("bf16", 1024, 1024, 1024), ("e4m3", 4096, 4096, 4096), ("s8", 8192, 8192, 8192),
                          ("s8", 8192, 1024, 8192), ("nvfp4", 8192, 28672, 8192), ("nvfp4", 8192, 3584, 8192),
                          ("mxfp4", 64, 57344, 8192), ("mxfp4", 64, 7168, 8192)]:
        lib, g = capi.bind(name, m, n, k, heuristic_config(name, m, n, k))
        plan = lib.plan(g)
        assert plan["grid"] <= 148 and plan["tiles"] >= 1
        if m <= 64:  # block-scaled fp4 decode: M on the padded 128-row side of fat single-CTA tiles
            assert (plan["swap"], plan["cta_group"], plan["tile_n"]) == (0, 1, 256)
    lib, g = capi.bind("e4m3", 16, 8192, 4096, heuristic_config("e4m3", 16, 8192, 4096))
    assert lib.plan(g)["swap"] == 1  # other formats: small M rides the MMA's N side


def test_plan_invariants_over_the_shape_suite():
    """For every format over every suite shape, the plan of the configuration
    gemm() would pick respects the hardware budget: shared memory within the
    227 KiB opt-in limit, tensor memory within 512 columns, at least two ring
    stages, accumulator and scale slots inside the allocation, and a TMA-store
    epilogue only on top of the staged one with 4-byte output."""
    from opengemm_b200 import capi
    from opengemm_b200.configs import heuristic_config, load_shapes
    from opengemm_b200.dtypes import DTYPES, NARROW_OUT, base_name

    checked = 0
    for name in list(DTYPES) + ["e4m3.bf16", "bf16.bf16", "tf32.f16"]:
        for m, n, k in load_shapes():
            try:
                lib, g = capi.bind(name, m, n, k, heuristic_config(base_name(name), m, n, k))
            except RuntimeError as exc:
                assert "multiple" in str(exc)
                continue
            p = lib.describe(g)
            assert p["smem_bytes"] <= 227 * 1024 and p["stages"] >= 2
            assert p["tmem_cols"] <= 512 and p["tmem_cols"] & (p["tmem_cols"] - 1) == 0
            assert p["sf_col"] + p["sf_slots"] * p["sf_cols"] <= p["tmem_cols"]
            assert p["acc_slots"] * p["acc_stride"] <= p["sf_col"] or p["sf_cols"] == 0
            assert p["stages"] * p["stage_bytes"] < p["smem_bytes"]
            assert p["tile_n"] % 16 == 0 and 16 <= p["tile_n"] <= 256
            assert p["num_tiles"] == p["tiles_m"] * p["tiles_n"] and 1 <= p["grid"] <= 148
            if p["epi_tma"]:
                assert p["epi_staged"] and p["tile_n"] % (128 // p["out_bytes"]) == 0  # whole 128-byte chunks
            assert p["out_bytes"] == (2 if (name in NARROW_OUT or DTYPES[base_name(name)].out is torch.bfloat16) else 4)
            checked += 1
    assert checked > 1000


def test_status_words_become_return_codes_with_a_readable_message():
    lib = capi.library("mm")
    assert lib.status(0) == capi.OG_OK
    assert lib.status(2 | (37 << 8)) == capi.OG_ERR_TIMEOUT
    assert "site 2" in lib.error() and "CTA 37" in lib.error()


def test_devices_beyond_the_table_are_refused_not_aliased():
    lib, g = capi.bind("bf16", 256, 256, 256, {"use_2cta": False, "output_n": 128})
    status = lib._launch(byref(g), 1, 1, 0, 0, 1, 64, 0)
    assert status == capi.OG_ERR_LAUNCH and "out of range" in lib.error()


def test_half_output_names_bind_to_the_two_byte_kernels():
    from opengemm_b200.dtypes import NARROW_OUT, base_name

    assert len(NARROW_OUT) == 18 and sum(name.endswith(".f16") for name in NARROW_OUT) == 9
    for name in ("bf16.f16", "e4m3xe5m2.f16"):
        lib, g = capi.bind(name, 512, 768, 1024, heuristic_config(base_name(name), 512, 768, 1024))
        described = lib.describe(g)
        assert described["out_bytes"] == 2 and 14 <= described["variant"] <= 19 and described["out"] == 3
