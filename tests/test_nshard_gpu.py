"""N-sharding on real GPUs: two ranks, one per GPU, each computes its column
shard of C with an ordinary gemm() on its rows of B; the all-gathered shards
must equal the oracle's unsharded product.  No collective is on the data path;
NCCL only gathers the result for the check.  Skipped with fewer than two GPUs."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import opengemm_oracle as ora
from tests.gemm_util import make_case, to_device

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, name, m, n, k, queue):
    import torch.distributed as dist

    import opengemm_b200 as og
    from opengemm_b200 import shard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        case = make_case(name, m, n, k, seed=12)
        d = og.DTYPES[name]
        a = to_device(case["a"], d.a)
        b_rows = shard.shard_rows(to_device(case["b"], d.b), world, rank).contiguous()
        sfa = sfb = None
        if d.impl == "smm":
            sfa = to_device(case["sfa"], d.sf)
            sfb = shard.shard_scales(to_device(case["sfb"], d.sf), name, n, k, world, rank)
        c_shard = shard.gemm_nshard(a, b_rows, sfa, sfb)
        full = shard.gather_columns(c_shard, n, world)
        torch.cuda.synchronize()
        got = full.view(torch.int16).cpu().numpy().view(np.uint16) if d.out is torch.bfloat16 else full.cpu().numpy()
        want = ora.reference(name, case["a"], case["b"], case.get("sfa_raw"), case.get("sfb_raw"))
        ok, _ = ora.check_close(name, k, got, want)
        strict, _ = ora.check_north_star(name, got, want)
        queue.put((rank, bool(ok and strict and got.shape == (m, n))))
    except Exception as exc:  # report at once; the parent must not wait out its timeout
        queue.put((rank, repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("name,shape", [("s8", (512, 1024, 1024)), ("nvfp4", (256, 1280, 1024)), ("e4m3", (300, 640, 512))])
def test_two_gpus_reassemble_the_full_product(name, shape):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, name, *shape, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results == [(0, True), (1, True)]
    assert [p.exitcode for p in procs] == [0, 0]
