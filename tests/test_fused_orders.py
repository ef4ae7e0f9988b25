"""Tile schedules of the fused GEMM + collective kernels, evaluated on the host by the same functions the kernels run."""
import ctypes
import itertools

import pytest


def _order(kind, rank, n, mb_per, tiles_n, group):
    from hcomm_b200 import _lib
    fn = _lib.load().HcommToolFusedTileOrder
    fn.restype = ctypes.c_int
    out = []
    for t in range(n * mb_per * tiles_n):
        mb, nb = ctypes.c_int(-1), ctypes.c_int(-1)
        assert fn(kind, rank, n, mb_per, tiles_n, group, t, ctypes.byref(mb), ctypes.byref(nb)) == 0
        out.append((mb.value, nb.value))
    return out


CASES = [(2, 16, 7, 8), (2, 16, 7, 1), (4, 8, 5, 5), (4, 8, 5, 3), (8, 4, 14, 2), (8, 4, 14, 1), (8, 4, 14, 4), (3, 5, 4, 2), (1, 6, 3, 4)]


@pytest.mark.parametrize("n,mb_per,tiles_n,group", CASES)
def test_reduce_scatter_order_visits_every_tile_once_remote_tiles_first(n, mb_per, tiles_n, group):
    everything = set(itertools.product(range(n * mb_per), range(tiles_n)))
    for rank in range(n):
        tiles = _order(0, rank, n, mb_per, tiles_n, group)
        assert len(tiles) == len(set(tiles)) and set(tiles) == everything
        owners = [mb // mb_per for mb, _ in tiles]
        remote = (n - 1) * mb_per * tiles_n
        assert all(o != rank for o in owners[:remote]) and all(o == rank for o in owners[remote:])
        # consecutive remote tiles go to consecutive destinations: the stores in flight spread over all peers
        for i in range(0, remote - (n - 1), n - 1) if n > 1 else []:
            assert sorted(owners[i:i + n - 1]) == sorted(set(range(n)) - {rank})
        # the owner consumes its tiles in the order every source produces them (flags are waited for in that order)
        own = [(mb % mb_per, nb) for mb, nb in tiles[remote:]]
        for src in range(n):
            if src == rank:
                continue
            made = [(mb % mb_per, nb) for mb, nb in _order(0, src, n, mb_per, tiles_n, group) if mb // mb_per == rank]
            assert made == own


@pytest.mark.parametrize("n,mb_per,tiles_n,group", CASES)
def test_all_gather_order_starts_with_own_rows_and_follows_the_arrival_of_blocks(n, mb_per, tiles_n, group):
    everything = set(itertools.product(range(n * mb_per), range(tiles_n)))
    for rank in range(n):
        tiles = _order(1, rank, n, mb_per, tiles_n, group)
        assert len(tiles) == len(set(tiles)) and set(tiles) == everything
        own = mb_per * tiles_n
        assert all(mb // mb_per == rank for mb, _ in tiles[:own]) and all(mb // mb_per != rank for mb, _ in tiles[own:])
        # blocks arrive block-major (block i of every source before block i + 1): a tile never needs a block of a later
        # group than the tiles after the next group boundary
        first_use = {}
        for pos, (mb, _) in enumerate(tiles[own:]):
            first_use.setdefault(mb % mb_per, pos)
        order_of_first_use = [b for b, _ in sorted(first_use.items(), key=lambda kv: kv[1])]
        groups = [b // group for b in order_of_first_use]
        assert groups == sorted(groups)


@pytest.mark.parametrize("n,mb_per,k", [(2, 8, 8192), (8, 8, 8192), (4, 3, 1000), (8, 2, 72), (3, 5, 16392)])
def test_all_gather_push_items_cover_every_byte_for_every_peer_once_block_by_block(n, mb_per, k):
    from hcomm_b200 import _lib
    fn = _lib.load().HcommToolFusedPushItem
    fn.restype = ctypes.c_int
    items = ctypes.c_int(0)
    assert fn(n, mb_per, k, -1, ctypes.byref(items), None, None, None, None) == 0
    block_bytes = 128 * k * 2
    covered = {p: [] for p in range(n - 1)}
    per_block = {}
    last_blk = 0
    for it in range(items.value):
        blk, peer = ctypes.c_int(), ctypes.c_int()
        off, ln = ctypes.c_ulonglong(), ctypes.c_ulonglong()
        assert fn(n, mb_per, k, it, None, ctypes.byref(blk), ctypes.byref(peer), ctypes.byref(off), ctypes.byref(ln)) == 0
        assert 0 <= peer.value < n - 1 and 0 <= blk.value < mb_per
        assert blk.value >= last_blk                      # block-major: the consumers take blocks in this order
        last_blk = blk.value
        assert off.value % 16 == 0 and ln.value % 16 == 0 and ln.value > 0
        assert off.value // block_bytes == blk.value and (off.value + ln.value - 1) // block_bytes == blk.value
        covered[peer.value].append((off.value, ln.value))
        per_block[(peer.value, blk.value)] = per_block.get((peer.value, blk.value), 0) + 1
    chunks = (block_bytes + (32 << 10) - 1) // (32 << 10)
    assert all(v == chunks for v in per_block.values()) and len(per_block) == (n - 1) * mb_per
    for p, ranges in covered.items():
        ranges.sort()
        pos = 0
        for off, ln in ranges:
            assert off == pos
            pos += ln
        assert pos == mb_per * block_bytes
