"""A host-side model of the work-unit enumeration of the CTA-pair GEMM (csrc/gemm_2cta.cu: ``unit_decode``,
``unit_krange`` and the launcher's choice between the plain and the hybrid cut of accumulating GEMMs).  The same
arithmetic in Python, checked exhaustively over many shapes: every (tile, k-block) is covered exactly once, whole
tiles are single units, and every pair of CTAs gets its whole-wave tiles before any tail slice."""
import pytest

PAIRS = 74          # 148 SMs
BM2, BN, BK = 256, 256, 64
OVERHEAD = 8


def choose(M, N, K):
    """(splits, full_tiles, tail_splits) as the launcher picks them for an fp32-accumulating GEMM."""
    tiles = -(-M // BM2) * -(-N // BN)
    kblocks = -(-K // BK)
    best = -(-tiles // PAIRS) * (kblocks + OVERHEAD)
    splits = 1
    s = 2
    while s <= 16 and s * 8 <= kblocks:
        cost = -(-(tiles * s) // PAIRS) * (-(-kblocks // s) + OVERHEAD)
        if cost * 100 < best * 97:
            best, splits = cost, s
        s += 1
    full = (tiles // PAIRS) * PAIRS
    tail = tiles - full
    full_tiles = tail_splits = 0
    if full > 0 and tail > 0:
        st = min(PAIRS // tail, 16)
        if st * 8 > kblocks:
            st = kblocks // 8
        if st >= 2:
            cost = (tiles // PAIRS) * (kblocks + OVERHEAD) + -(-(tail * st) // PAIRS) * (-(-kblocks // st) + OVERHEAD)
            if cost * 100 < best * 99:
                splits, full_tiles, tail_splits = 1, full, st
    return tiles, kblocks, splits, full_tiles, tail_splits


def decode(u, tiles, splits, full_tiles, tail_splits):
    if tail_splits > 0:
        if u < full_tiles:
            return u, 0, 1
        v, tail = u - full_tiles, tiles - full_tiles
        return full_tiles + v % tail, v // tail, tail_splits
    return u % tiles, u // tiles, splits


def krange(sp, kblocks, nsp):
    return sp * kblocks // nsp, (sp + 1) * kblocks // nsp


SHAPES = [(4096, 2560, 16384), (2560, 2048, 16384), (2560, 10240, 16384), (20480, 2560, 16384), (4096, 2560, 262144),
          (262144, 2560, 4096), (1024, 512, 4096), (256, 256, 64), (4104, 2312, 4096), (18944, 256, 512),
          (3072, 4096, 16384), (14336, 4096, 8192)]
SHAPES += [(256 * a, 256 * b, 64 * c) for a in (1, 3, 9, 10) for b in (1, 8, 15) for c in (1, 16, 200)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_every_tile_and_k_block_is_covered_exactly_once(M, N, K):
    tiles, kblocks, splits, full_tiles, tail_splits = choose(M, N, K)
    units = full_tiles + (tiles - full_tiles) * tail_splits if tail_splits else tiles * splits
    seen = {}
    for u in range(units):
        tile, sp, nsp = decode(u, tiles, splits, full_tiles, tail_splits)
        kb0, kb1 = krange(sp, kblocks, nsp)
        assert 0 <= tile < tiles and 0 <= kb0 < kb1 <= kblocks   # no empty unit: an empty one would hand the
        for kb in range(kb0, kb1):                                # epilogue an accumulator nobody wrote
            assert (tile, kb) not in seen
            seen[(tile, kb)] = u
        if tail_splits and tile < full_tiles:
            assert (kb0, kb1) == (0, kblocks)                     # whole tiles are single units (plain RMW epilogue)
    assert len(seen) == tiles * kblocks


@pytest.mark.parametrize("M,N,K", [s for s in SHAPES if choose(*s)[4] > 0])
def test_whole_waves_come_before_the_tail_on_every_cta_pair(M, N, K):
    tiles, kblocks, splits, full_tiles, tail_splits = choose(M, N, K)
    units = full_tiles + (tiles - full_tiles) * tail_splits
    pairs = min(units, PAIRS)
    assert full_tiles % PAIRS == 0 and 0 < tiles - full_tiles < PAIRS
    for p in range(pairs):
        kinds = [decode(u, tiles, splits, full_tiles, tail_splits)[2] == 1 for u in range(p, units, pairs)]
        assert kinds == sorted(kinds, reverse=True)               # True (whole tile) first, then tail slices
        assert sum(kinds) == full_tiles // PAIRS


def test_the_benchmark_shapes_take_the_hybrid_cut():
    assert choose(4096, 2560, 16384)[3:] == (148, 6)     # qkv weight gradient: 160 tiles = 2 waves + 12 tiles cut in 6
    assert choose(2560, 2048, 16384)[3:] == (74, 12)     # o weight gradient
    assert choose(2560, 10240, 16384)[3:] == (370, 2)    # down-projection weight gradient
    assert choose(20480, 2560, 16384)[2:] == (1, 0, 0)   # gate|up: 800 tiles, tail of 60 cannot be cut usefully
