"""The five tile orders (OgGemm.walk, numbered like the reference's
opengemm/src/mm/types.cuh:78-84): on the CPU, every order visits every tile of
a grid exactly once and keeps the locality it is named for; on the GPU, a GEMM
gives the same product whichever order its tiles are visited in."""

import pytest
import torch

from opengemm_b200 import capi
from tests.gemm_util import assert_parity, make_case, run_library

WALKS = {"bands": 0, "serpentine": 1, "blocks": 2, "hilbert": 3, "row bands": 4}


def order_of(m, n, walk, group, output_n=128, use_2cta=False):
    lib, g = capi.bind("bf16", m, n, 256, {"use_2cta": use_2cta, "output_n": output_n, "walk": walk,
                                           "supergroup": group, "cluster_m": 2 if use_2cta else 1})
    return lib.tile_order(g), lib.plan(g)


@pytest.mark.parametrize("walk", WALKS.values(), ids=WALKS.keys())
@pytest.mark.parametrize("shape", [(128, 128), (1024, 1024), (1280, 4224), (8192, 640), (3000, 2000), (128, 9000)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("group", [1, 3, 8, 64])
def test_every_order_visits_every_tile_once(walk, shape, group):
    m, n = shape
    order, plan = order_of(m, n, walk, group)
    tiles_m, tiles_n = -(-m // plan["tile_m"]), -(-n // plan["tile_n"])
    assert len(order) == tiles_m * tiles_n == plan["tiles"]
    assert sorted(order) == [(i, j) for i in range(tiles_m) for j in range(tiles_n)]


def test_orders_keep_their_locality():
    order, _ = order_of(2048, 4096, WALKS["bands"], 4)          # 16 x 32 tiles
    assert order[:5] == [(0, 0), (0, 1), (0, 2), (0, 3), (1, 0)]
    serpentine, _ = order_of(2048, 4096, WALKS["serpentine"], 4)
    assert serpentine[:64] == order[:64]                         # first band alike ...
    assert serpentine[64] == (15, 4) and serpentine[127] == (0, 7)  # ... the second walked back up
    rows, _ = order_of(2048, 4096, WALKS["row bands"], 4)
    assert rows[:5] == [(0, 0), (1, 0), (2, 0), (3, 0), (0, 1)]
    blocks, _ = order_of(2048, 4096, WALKS["blocks"], 4)
    assert blocks[:5] == [(0, 0), (1, 0), (2, 0), (3, 0), (0, 1)] and blocks[16] == (4, 0)
    hilbert, _ = order_of(2048, 4096, WALKS["hilbert"], 1)
    steps = [abs(a[0] - b[0]) + abs(a[1] - b[1]) for a, b in zip(hilbert, hilbert[1:])]
    assert max(steps) <= 2 and steps.count(1) >= len(steps) - 2  # a continuous curve (a diagonal step only where a side is odd)


@pytest.mark.gpu
@pytest.mark.parametrize("walk", [1, 2, 3, 4], ids=["serpentine", "blocks", "hilbert", "row bands"])
@pytest.mark.parametrize("name,shape,knobs", [
    ("bf16", (1280, 2176, 512), dict(use_2cta=True, output_n=128, supergroup=3)),
    ("s8", (2304, 2560, 1024), dict(use_2cta=False, output_n=96, supergroup=4)),
    ("e4m3", (640, 8200, 256), dict(use_2cta=True, output_n=256, supergroup=2, use_clc=True)),
], ids=["bf16-pair", "s8-single", "e4m3-clc"])
def test_the_product_does_not_depend_on_the_order(walk, name, shape, knobs):
    m, n, k = shape
    case = make_case(name, m, n, k, seed=17)
    config = dict({"swap_ab": False, "epi_direct": 0, "cluster_m": 2 if knobs["use_2cta"] else 1, "walk": walk}, **knobs)
    assert_parity(case, run_library(case, config))
