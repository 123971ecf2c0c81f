"""N-sharding of one GEMM across the GPUs of a box: C[:, n0:n1] = A . B[n0:n1, :]^T.

B, its scales and C are split along N on 128-row boundaries (so a shard of the
128x4 blocked scale buffer is itself a valid blocked buffer); A and its
scales are replicated.  Every shard is an independent GEMM: no collective is
on the data path.  `gather_columns` is for callers (and tests) that want the
full C back.  The reference has no multi-GPU path; this is the partitioning
its operands' layout admits without any reduction.
"""

import torch

from .dtypes import DTYPES, sf_block

ALIGN = 128


def shard_bounds(n, world, rank, align=ALIGN):
    """Rows `[n0, n1)` of B (columns of C) that `rank` of `world` owns.

    Blocks of `align` rows are dealt out as evenly as possible, the first
    `blocks % world` ranks taking one more; the last block may be ragged.
    """
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} is not in a world of {world}")
    blocks = -(-n // align)
    base, extra = divmod(blocks, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return min(first * align, n), min((first + count) * align, n)


def shard_rows(b, world, rank):
    """This rank's rows of B (a view; contiguous because rows are K-major)."""
    n0, n1 = shard_bounds(b.size(0), world, rank)
    return b[n0:n1]


def shard_scales(sfb, name, n, k, world, rank):
    """This rank's part of B's blocked scale buffer: whole 128-row blocks, each
    `ceil(K / (4 * block))` atoms of 512 bytes, contiguous in the flat buffer."""
    d = DTYPES[name]
    n0, n1 = shard_bounds(n, world, rank)
    atoms_per_block = -(-k // (4 * sf_block(d)))
    flat = sfb.reshape(-1)
    return flat[(n0 // ALIGN) * atoms_per_block * 512 : -(-n1 // ALIGN) * atoms_per_block * 512]


def gemm_nshard(a, b_shard, sfa=None, sfb_shard=None, out=None, **names):
    """The local shard of C: an ordinary gemm() on this rank's rows of B."""
    from .api import gemm

    return gemm(a, b_shard, sfa, sfb_shard, out=out, **names)


def gather_columns(c_shard, n, world, group=None):
    """All-gather the column shards into the full row-major `[M, n]` C on every rank."""
    import torch.distributed as dist

    m = c_shard.size(0)
    widths = [shard_bounds(n, world, r)[1] - shard_bounds(n, world, r)[0] for r in range(world)]
    widest = max(widths)
    padded = c_shard.new_zeros((m, widest))
    padded[:, : c_shard.size(1)] = c_shard
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([part[:, :w] for part, w in zip(parts, widths)], dim=1)
