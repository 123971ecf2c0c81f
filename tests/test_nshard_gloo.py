"""The N-sharded path with two CPU ranks over gloo: each rank takes its rows of
B (and its slice of the blocked scales), forms its column shard of C, and the
gathered shards equal the unsharded product.  The per-rank product is taken
with the CPU oracle here; on GPUs it is one ordinary gemm() per rank."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from opengemm_b200 import shard
from oracle import opengemm_oracle as ora
from tests.gemm_util import make_case


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, name, m, n, k, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = make_case(name, m, n, k, seed=5)
        n0, n1 = shard.shard_bounds(n, world, rank)
        b_rows = shard.shard_rows(torch.from_numpy(case["b"]), world, rank).numpy()
        assert b_rows.shape[0] == n1 - n0
        sfb_raw = None
        if "sfb" in case:
            part = shard.shard_scales(torch.from_numpy(case["sfb"]), name, n, k, world, rank).numpy()
            sfb_raw = ora.from_blocked(part, n1 - n0, case["sfb_raw"].shape[1])
            assert np.array_equal(sfb_raw, case["sfb_raw"][n0:n1])
        c_local = ora.reference(name, case["a"], b_rows, case.get("sfa_raw"), sfb_raw)
        c_local = torch.from_numpy(c_local.astype(np.int32) if c_local.dtype == np.uint16 else c_local)
        full = shard.gather_columns(c_local, n, world)
        want = ora.reference(name, case["a"], case["b"], case.get("sfa_raw"), case.get("sfb_raw"))
        want = want.astype(np.int32) if want.dtype == np.uint16 else want
        ok = full.shape == (m, n) and np.array_equal(full.numpy(), want)
        queue.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,shape", [("s8", (48, 384, 256)), ("nvfp4", (40, 520, 256)), ("bf16", (33, 300, 128))])
def test_two_ranks_reassemble_the_full_product(name, shape):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, name, *shape, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]
