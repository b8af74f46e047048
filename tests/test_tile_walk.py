"""The tile enumeration of the fused launches, evaluated on the host through the C ABI.

Every rank's CTAs take output tiles in the order ``edm_tile_walk`` reports.  The protocol relies
on three properties, checked here for every mode, world size and a set of ragged shapes:
each rank produces every tile exactly once; all ranks agree on which rank owns a tile and on the
slot (index among the owner's tiles) its partials land in; and slots of one owner are distinct.
"""
import itertools

import pytest

from edmir_b200 import symm

SHAPES = [(8192, 8192), (8192, 1280), (2048, 7168), (1024, 256), (4096, 300), (1536, 2304), (256, 256)]


def _blocks(M, N, tile_m, tile_n):
    return -(-M // tile_m), -(-N // tile_n)


@pytest.mark.parametrize("tile_m", [128, 256])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("op", ["gemm", "gemm_rs", "gemm_ar", "ag_gemm"])
def test_every_tile_once_and_ranks_agree(native_lib, op, world, tile_m):
    for (M, N), (band, cols), units in itertools.product(SHAPES, ((0, 0), (8, 0), (8, 9), (4, 3), (0, 5)), (1, 37, 148)):
        if op == "gemm" and world > 1:
            continue
        if op == "gemm_rs" and (M % world or (M // world) % tile_m):
            continue
        mb, nb = _blocks(M, N, tile_m, 256)
        owners: dict = {}
        for rank in range(world):
            walk = symm.tile_walk(op, rank, world, M, N, tile_m, 256, band, units, cols)
            tiles = [(m, n) for m, n, _, _ in walk if m >= 0]
            assert sorted(tiles) == sorted(itertools.product(range(mb), range(nb))), (op, world, M, N, rank)
            if op == "gemm_ar" and world > 1:
                assert len(walk) % world == 0 and len(walk) - len(tiles) < world
            else:
                assert len(walk) == len(tiles)
            for m, n, owner, idx in walk:
                if m < 0:
                    continue
                if op in ("gemm_rs", "gemm_ar") and world > 1:
                    assert owners.setdefault((m, n), (owner, idx)) == (owner, idx)
                else:
                    assert owner == rank
        if owners:
            per_owner: dict = {}
            for (m, n), (owner, idx) in owners.items():
                per_owner.setdefault(owner, []).append(idx)
                if op == "gemm_rs":
                    assert owner == m // (mb // world)
            for owner, idxs in per_owner.items():
                assert sorted(idxs) == list(range(len(idxs))), (op, world, M, N, owner)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_reduce_walk_sends_to_every_peer_each_round_and_ends_on_own_tiles(native_lib, world):
    M, N, units = 8192, 8192, 74
    for op in ("gemm_rs", "gemm_ar"):
        for rank in range(world):
            walk = symm.tile_walk(op, rank, world, M, N, 256, 256, 0, units)
            rounds = len(walk) // world
            defer = min(rounds, units)
            head = walk[:(rounds - defer) * world]
            for r in range(rounds - defer):
                # every round reaches every owner once, starting at a position that rotates with the round
                assert [o for _, _, o, _ in head[r * world:(r + 1) * world]] == \
                    [(rank + 1 + (d + r) % world) % world for d in range(world)]
            # a unit (every units-th position) therefore alternates between owners: with a fixed
            # order and an even unit count it would only ever meet one parity class of them
            for u in (0, 1):
                mine = [o for _, _, o, _ in head[u::units]]
                if len(mine) >= 4:
                    assert {(o - rank) % 2 for o in mine} == {0, 1}, (op, rank, u, mine)
            tail = walk[-defer:]
            assert all(o == rank for _, _, o, _ in tail)
            middle = walk[(rounds - defer) * world:len(walk) - defer]
            assert all(o != rank for _, _, o, _ in middle)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_gather_walk_follows_arrival_order(native_lib, world):
    M, N, tile_m = 8192, 7168, 256
    per_rank = M // world // tile_m
    for rank in range(world):
        walk = symm.tile_walk("ag_gemm", rank, world, M, N, tile_m, 256, 0, 74)
        shard_of = [((m - rank * per_rank) % (M // tile_m)) // per_rank for m, _, _, _ in walk]
        assert all(s == 0 for s in shard_of[:min(per_rank, 16)])      # first tiles: own rows
        if per_rank < 16:
            # a shard shorter than a band is a band of its own: every tile of the own shard comes
            # before any tile whose rows have to arrive first
            own = per_rank * (N // 256)
            assert all(s == 0 for s in shard_of[:own]) and shard_of[own] == 1
        # position of the first tile of shard s (in arrival order s = 0 own, 1 = rank+1, ...)
        first = {s: shard_of.index(s) for s in range(world)}
        assert [first[s] for s in range(world)] == sorted(first.values())
        # over the first four shards a shard is started only when the shard two places earlier
        # (which arrived two transfers earlier) is finished
        last = {s: len(shard_of) - 1 - shard_of[::-1].index(s) for s in range(world)}
        for s in range(2, min(world, 4)):
            assert first[s] > last[s - 2]


def test_split_of_the_last_wave(native_lib):
    # the layer's shapes on 74 CTA pairs (K blocks of 64 bf16)
    assert symm.tail_split(32 * 5, 74, 128) == (148, 12, 4)      # qkv: 160 tiles, third wave of 12
    assert symm.tail_split(32 * 28, 74, 128) == (888, 8, 8)      # gate_up: 896 tiles, last wave of 8
    assert symm.tail_split(32 * 32, 74, 56) == (1024, 0, 1)      # down: last wave of 62, left alone
    assert symm.tail_split(32 * 32, 74, 16) == (1024, 0, 1)      # o_proj: K too short to cut
    assert symm.tail_split(20, 74, 128) == (0, 20, 2)            # less than one wave: every tile is cut
    assert symm.tail_split(16, 148, 112) == (0, 16, 8)           # decode-sized GEMM: split-K over idle CTAs
    assert symm.tail_split(16, 148, 28) == (16, 0, 1)            # K too short for the exchange to pay
    for tiles in range(1, 400, 7):
        for units in (1, 2, 37, 74, 148):
            for kb in (1, 8, 16, 31, 32, 40, 128, 448):
                first, split, parts = symm.tail_split(tiles, units, kb)
                assert first + split == tiles
                assert parts in (1, 2, 4, 8)
                if parts > 1:
                    assert first % units == 0                         # whole waves before the tail
                    assert split * parts <= units                     # one piece per unit at most
                    assert kb >= 32 and kb // parts >= 4              # every piece has work to do
                    # the pieces' K ranges tile [0, kb) without gaps
                    edges = [kb * p // parts for p in range(parts + 1)]
                    assert edges[0] == 0 and edges[-1] == kb and all(a < b for a, b in zip(edges, edges[1:]))
                else:
                    assert split == 0


def test_bad_arguments(native_lib):
    with pytest.raises(ValueError):
        symm.tile_walk("gemm_rs", 2, 2, 1024, 1024)
    with pytest.raises(ValueError):
        symm.tile_walk("gemm_rs", 0, 2, 1024 + 128, 1024)   # rows per rank not on tile edges


def test_launch_plans_of_the_layer_and_of_decode_shapes(native_lib):
    from edmir_b200 import linear
    plan = lambda *shape: tuple(linear.gemm_plan(*shape).values())   # (cta_group, block_n, ctas, pieces)
    # prefill layer at 8192 tokens: CTA pairs on every SM; qkv and gate_up cut their last wave
    assert plan(8192, 1280, 8192) == (2, 256, 148, 4)
    assert plan(8192, 7168, 8192) == (2, 256, 148, 8)
    assert plan(8192, 8192, 1024) == (2, 256, 148, 1)
    assert plan(8192, 8192, 3584) == (2, 256, 148, 1)
    # decode rows of the 8B down_proj.  Up to 64 tokens: the decode kernel, 32 tiles of 128 columns
    # each cut into 4 pieces along K (one cluster per tile); 8 tiles are cut into 8; more tiles than
    # fit twice are not cut; more tiles than SMs take the general kernel
    assert plan(16, 4096, 14336) == (1, 128, 128, 4)
    assert plan(1, 4096, 1792) == (1, 128, 128, 4)
    assert plan(32, 1024, 8192) == (1, 128, 64, 8)
    assert plan(8, 16384, 512) == (1, 128, 128, 1)
    assert plan(8, 32768, 512)[1] != 128
    assert plan(64, 4096, 7168) == (1, 128, 128, 4)
    assert plan(65, 4096, 7168) == (1, 256, 128, 8)
    # 128 tokens: split-K over 128 CTAs for long K, narrow tiles for short K
    assert plan(128, 4096, 7168) == (1, 256, 128, 8)
    assert plan(128, 4096, 1792) == (1, 32, 128, 1)
    # 64 pair tiles on 74 pairs: nothing to cut
    assert plan(1024, 4096, 3584) == (2, 256, 128, 1)
    with pytest.raises(ValueError):
        linear.gemm_plan(0, 16, 16)
