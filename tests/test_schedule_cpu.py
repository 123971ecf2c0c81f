"""The stream-K work schedule, modelled on the CPU.

`schedule` restates WorkIter of opengemm_b200/csrc/kernel.cuh: whole waves of
tiles dealt out statically, the tiles of the partial wave cut along K into
equal contiguous unit ranges.  The properties the kernel relies on are
checked for many (tiles, clusters, K-blocks) combinations: every K block of
every tile is computed exactly once; a cluster contributes (starts inside a
tile) at most once; and the finisher of a shared tile finds exactly the
clusters that contribute to it, skipping those whose range is empty."""

import pytest


def schedule(tiles, grid_clusters, k_blocks, ways=None):
    """`ways`: at most that many clusters share one leftover tile (None: all clusters share the wave)."""
    static_tiles = (tiles // grid_clusters) * grid_clusters
    total = (tiles - static_tiles) * k_blocks
    clusters = grid_clusters if ways is None else min(grid_clusters, (tiles - static_tiles) * min(ways, k_blocks))
    per_cluster = []
    for c in range(grid_clusters):
        work = [(t, 0, k_blocks) for t in range(c, static_tiles, grid_clusters)]
        shares = c < clusters
        u, u_end = (total * c // clusters, total * (c + 1) // clusters) if shares else (0, 0)
        while u < u_end:
            t = u // k_blocks
            kb0 = u - t * k_blocks
            left = u_end - u
            kb1 = kb0 + left if left < k_blocks - kb0 else k_blocks
            work.append((static_tiles + t, kb0, kb1))
            u += kb1 - kb0
        per_cluster.append(work)
    return per_cluster, static_tiles, total, clusters


def sharers_found_by_finisher(c, tile, clusters, k_blocks, static_tiles, total):
    tile_end = (tile - static_tiles + 1) * k_blocks
    found, j = [], c + 1
    while j < clusters and total * j // clusters < tile_end:
        if total * (j + 1) // clusters > total * j // clusters:  # has_work
            found.append(j)
        j += 1
    return found


@pytest.mark.parametrize("tiles,clusters,k_blocks", [
    (448, 148, 32), (90, 74, 4), (4, 148, 64), (56, 148, 32), (180, 74, 4), (6, 74, 32), (512, 148, 1),
    (256, 74, 32), (128, 74, 64), (1, 148, 128), (149, 148, 2), (147, 148, 3), (1024, 74, 128), (7, 3, 5),
])
@pytest.mark.parametrize("ways", [None, 2, 4])
def test_schedule_covers_every_unit_once_and_pairs_finishers_with_contributors(tiles, clusters, k_blocks, ways):
    work, static_tiles, total, clusters = schedule(tiles, clusters, k_blocks, ways)
    seen = {}
    for c, items in enumerate(work):
        assert sum(1 for _, kb0, _ in items if kb0 > 0) <= 1, "a cluster contributes at most once"
        for tile, kb0, kb1 in items:
            assert 0 <= kb0 < kb1 <= k_blocks
            for kb in range(kb0, kb1):
                seen[(tile, kb)] = seen.get((tile, kb), 0) + 1
    assert len(seen) == tiles * k_blocks and set(seen.values()) == {1}
    for c, items in enumerate(work):
        for tile, kb0, kb1 in items:
            if kb0 == 0 and kb1 < k_blocks:  # this cluster finishes a shared tile
                found = sharers_found_by_finisher(c, tile, clusters, k_blocks, static_tiles, total)
                contributors = [j for j, other in enumerate(work) for t, a, _ in other if t == tile and a > 0]
                assert found == contributors


def test_staged_epilogue_addressing_is_a_bijection_without_bank_conflicts():
    """Python model of the staged output path of the kernel's epilogue
    (store_staged in csrc/kernel.cuh): lane L writes its row's eight 16-byte
    units to row L of a 32 x 128-byte buffer at unit u ^ (L % 8); the warp then
    reads row r = 4 i + L // 8, unit L % 8 back from unit (L % 8) ^ (r % 8).
    Every (row, unit) must be written once, read once, and come back as the
    unit it was written as; and the eight lanes that share a shared-memory
    wavefront (a quarter warp moves 8 x 16 bytes = 128 bytes = all 32 banks)
    must touch eight different 16-byte bank groups."""
    buffer = {}
    for lane in range(32):
        for u in range(8):
            address = lane * 128 + ((u ^ (lane & 7)) << 4)
            assert address not in buffer
            buffer[address] = (lane, u)  # row, logical unit
    assert len(buffer) == 256
    for u in range(8):  # one st.shared.v4 per unit index: quarter warps of eight lanes
        for quarter in range(4):
            groups = {((lane * 128 + ((u ^ (lane & 7)) << 4)) >> 4) % 8 for lane in range(8 * quarter, 8 * quarter + 8)}
            assert len(groups) == 8
    seen = set()
    for i in range(8):
        for lane in range(32):
            sub_row, unit = lane >> 3, lane & 7
            r = 4 * i + sub_row
            row, logical = buffer[r * 128 + ((unit ^ (r & 7)) << 4)]
            assert (row, logical) == (r, unit)  # the 16 bytes this lane stores belong to row r, columns of `unit`
            seen.add((r, unit))
        for quarter in range(4):  # reads: the same no-conflict property
            groups = set()
            for lane in range(8 * quarter, 8 * quarter + 8):
                r = 4 * i + (lane >> 3)
                groups.add(((r * 128 + (((lane & 7) ^ (r & 7)) << 4)) >> 4) % 8)
            assert len(groups) == 8
    assert len(seen) == 256
