"""CPU tests of the GEMM's host-side launch plan (tile grid, K splits, stream-K partition, raster): the same
C++ functions the kernel runs are enumerated through the C ABI, no GPU involved."""
import ctypes

import pytest


def _plan(L, M, N, K, bn, cg, sk, max_ctas=0, sms=148, tf32=0):
    out = (ctypes.c_uint32 * 10)()
    rc = L.spork_gemm_sm100_plan(M, N, K, bn, cg, sk, max_ctas, sms, tf32, out)
    assert rc == 0
    keys = ["tiles_m", "tiles_n", "num_kb", "split_k", "kb_per_split", "groups", "dp_tiles", "sk_tiles", "sk_share",
            "sk_extra"]
    return dict(zip(keys, list(out)))


def _items(L, M, N, K, bn, cg, sk, group, max_ctas=0, sms=148, tf32=0):
    cap = 4096
    buf = (ctypes.c_uint32 * (5 * cap))()
    n = L.spork_gemm_sm100_plan_items(M, N, K, bn, cg, sk, max_ctas, sms, tf32, group, buf, cap)
    assert 0 <= n <= cap
    return [tuple(buf[5 * i:5 * i + 5]) for i in range(n)]


@pytest.fixture(scope="module")
def L(sp):
    lib = sp.lib()
    u32, i32 = ctypes.c_uint32, ctypes.c_int
    lib.spork_gemm_sm100_plan.argtypes = [u32, u32, u32, i32, i32, i32, i32, i32, i32, ctypes.POINTER(u32)]
    lib.spork_gemm_sm100_plan.restype = i32
    lib.spork_gemm_sm100_plan_items.argtypes = [u32, u32, u32, i32, i32, i32, i32, i32, i32, u32, ctypes.POINTER(u32), u32]
    lib.spork_gemm_sm100_plan_items.restype = i32
    return lib


def test_headline_plan(L):
    p = _plan(L, 8192, 8192, 8192, 256, 2, 1)
    assert (p["tiles_m"], p["tiles_n"], p["num_kb"], p["groups"]) == (32, 32, 128, 74)
    assert p["split_k"] == 1 and p["sk_tiles"] == 0
    p = _plan(L, 16384, 64, 8192, 64, 2, 1)
    assert (p["tiles_m"], p["tiles_n"], p["groups"]) == (64, 1, 64)  # fewer tiles than CTA pairs
    p = _plan(L, 8192, 8192, 8192, 256, 2, 1, tf32=1)
    assert p["num_kb"] == 256  # 32 fp32 elements per 128-byte row


def test_split_k_is_normalised(L):
    p = _plan(L, 512, 512, 2048, 128, 2, 1000)
    assert p["num_kb"] == 32 and p["split_k"] == 32 and p["kb_per_split"] == 1
    p = _plan(L, 512, 512, 2048, 128, 2, 3)
    assert p["kb_per_split"] == 11 and p["split_k"] == 3  # 11 + 11 + 10, no empty split
    assert L.spork_gemm_sm100_plan(1, 1, 8, 100, 2, 1, 0, 148, 0, (ctypes.c_uint32 * 10)()) == 10001
    assert L.spork_gemm_sm100_plan(1, 1, 8, 512, 2, -1, 0, 148, 0, (ctypes.c_uint32 * 10)()) == 10001  # no stream-K with 256 x 512 tiles


@pytest.mark.parametrize("shape,bn,cg,sk,max_ctas", [
    ((8192, 8192, 8192), 256, 2, 1, 0), ((1536, 2304, 65536), 256, 2, -1, 0), ((16384, 64, 8192), 64, 2, -1, 0),
    ((160, 480, 816), 128, 1, -1, 0), ((2048, 6000, 264), 64, 2, -1, 20), ((1000, 264, 136), 256, 2, 1, 0),
    ((768, 768, 4096), 256, 1, 4, 0), ((300, 131, 2056), 128, 2, -1, 0), ((8192, 8192, 8192), 256, 2, -1, 0),
    ((4096, 4096, 64), 128, 2, 3, 6), ((4096, 4096, 4096), 256, 2, -1, 0), ((2304, 2816, 65536), 256, 2, -1, 0),
    ((2048, 2048, 2048), 256, 2, -1, 0), ((512, 768, 1024), 256, 2, -1, 0),
    # 256 x 512 tiles, and split-K with K fastest in the schedule (gemm_sm90_k_mode::split_k_inner)
    ((8192, 8192, 8192), 512, 2, 1, 0), ((1000, 2050, 264), 512, 2, 3, 4), ((640, 1100, 2048), 256, 1, -3, 6),
    ((1536, 2304, 8192), 512, 2, -4, 0),
])
def test_every_k_block_of_every_tile_is_covered_exactly_once(L, shape, bn, cg, sk, max_ctas):
    M, N, K = shape
    p = _plan(L, M, N, K, bn, cg, sk, max_ctas)
    covered = {}
    reduce_tiles = set()
    for g in range(p["groups"]):
        for (m, n, kb0, kb1, red) in _items(L, M, N, K, bn, cg, sk, g, max_ctas):
            assert m < p["tiles_m"] and n < p["tiles_n"] and kb0 < kb1 <= p["num_kb"]
            if red:
                reduce_tiles.add((m, n))
            for kb in range(kb0, kb1):
                assert (m, n, kb) not in covered, "K block computed twice"
                covered[(m, n, kb)] = (g, red)
    assert len(covered) == p["tiles_m"] * p["tiles_n"] * p["num_kb"]
    # a tile is either stored whole by one group or reduce-added by all of its contributors, never mixed
    for (m, n, kb), (g, red) in covered.items():
        assert bool(red) == ((m, n) in reduce_tiles)
    if sk == 1:
        assert not reduce_tiles
    if sk <= -2:
        # K fastest: the ranges of one tile sit next to each other in the work list, i.e. on neighbouring groups
        first = _items(L, M, N, K, bn, cg, sk, 0, max_ctas)[0]
        if p["groups"] > 1:
            second = _items(L, M, N, K, bn, cg, sk, 1, max_ctas)[0]
            assert first[:2] == second[:2] and second[2] == first[3]
    if p["sk_tiles"]:
        # stream-K: the tail tiles (fewer than groups) are cut into aligned K ranges, at most one per group
        assert len(reduce_tiles) == p["sk_tiles"] < p["groups"] or p["dp_tiles"] == 0
        assert p["sk_tiles"] * p["sk_extra"] <= p["groups"] and p["sk_extra"] >= 2
        starts = set()
        for g in range(p["groups"]):
            red_items = [it for it in _items(L, M, N, K, bn, cg, sk, g, max_ctas) if it[4]]
            assert len(red_items) <= 1
            for (_, _, kb0, kb1, _) in red_items:
                assert kb0 % p["sk_share"] == 0 and kb1 - kb0 <= p["sk_share"]
                starts.add(kb0)
        assert len(starts) == p["sk_extra"]  # every tile is cut at the same K offsets
    elif sk == -1:
        assert not reduce_tiles  # a tail that is more than half a wave runs whole


def test_raster_keeps_concurrent_tiles_compact(L):
    """Tiles that run in the same wave span 8 m-tiles and a short run of n-tiles (the superblock raster)."""
    firsts = [_items(L, 8192, 8192, 8192, 256, 2, 1, g)[0][:2] for g in range(74)]
    ms = {m for m, _ in firsts}
    ns = {n for _, n in firsts}
    assert ms == set(range(8)) and len(ns) <= 10


def test_automatic_split_fills_the_waves(L):
    """split_k = 0 leaves the count to the library: 1 when the tiles fill the machine or K is short, else the
    count that makes the best use of the waves (the reference's huge-K shapes, gemm/gemm_main.cpp:111-117)."""
    assert _plan(L, 8192, 8192, 8192, 256, 2, 0)["split_k"] == 1          # 1024 tiles for 74 CTA pairs
    assert _plan(L, 512, 512, 512, 256, 2, 0)["split_k"] == 1             # 8 K blocks: too short to cut
    assert _plan(L, 16384, 64, 8192, 64, 2, 0)["split_k"] == 1            # narrow tiles: bound by memory
    p = _plan(L, 1536, 2304, 65536, 256, 2, 0)                             # 54 tiles: 4 x 54 = 216 items = 2.92 waves
    assert p["split_k"] == 4 and p["kb_per_split"] == 256
    p = _plan(L, 1024, 2816, 49152, 256, 2, 0)                             # 44 tiles: 5 x 44 = 220 items = 2.97 waves
    assert p["split_k"] == 5
    p = _plan(L, 512, 512, 16384, 256, 2, 0)                               # 4 tiles: as many ranges as allowed
    assert p["split_k"] == 16 and p["kb_per_split"] == 16
    # every K block of every tile is still covered exactly once
    seen = {}
    p = _plan(L, 1024, 2816, 49152, 256, 2, 0)
    for g in range(p["groups"]):
        for (m, n, k0, k1, reduce) in _items(L, 1024, 2816, 49152, 256, 2, 0, g):
            assert reduce == 1
            for kb in range(k0, k1):
                assert (m, n, kb) not in seen
                seen[(m, n, kb)] = True
    assert len(seen) == p["tiles_m"] * p["tiles_n"] * p["num_kb"]


def test_tile_choice_of_the_default_entry_point(sp):
    """What a launch resolves to, without a GPU: width from N for skinny problems (two column blocks per stage
    when K is long), single CTAs for tiny latency-bound ones, 256 x 512 pair tiles for large deep problems whose
    waves they fill as well as 256 x 256 tiles do."""
    c = sp.choice
    assert c(8192, 8192, 8192) == {"block_n": 512, "cta_group": 2, "k_atoms": 1, "split_k": 1}
    assert c(65536, 8192, 8192)["block_n"] == 512 and c(40016, 32768, 6400)["block_n"] == 512
    assert c(8192, 8192, 2048)["block_n"] == 256          # short K: the tile ends would cost more than the bytes save
    assert c(4096, 4096, 4096)["block_n"] == 256          # 128 wide tiles: less than two waves
    assert c(15360, 1536, 8192)["block_n"] == 256         # 180 wide tiles = 2.4 waves (three), 360 narrow = 4.9 (five)
    assert c(7680, 3072, 16384)["block_n"] == 256
    assert c(8192, 8200, 8192)["block_n"] == 256          # 8200 columns would pad the last tile column to 8704
    for n in (64, 128):
        assert c(16384, n, 8192) == {"block_n": n, "cta_group": 2, "k_atoms": 2, "split_k": 1}
    assert c(16384, 256, 8192) == {"block_n": 256, "cta_group": 2, "k_atoms": 1, "split_k": 1}
    assert c(160, 480, 816) == {"block_n": 128, "cta_group": 1, "k_atoms": 1, "split_k": 1}
    assert c(256, 256, 512)["cta_group"] == 1
    assert c(8192, 8192, 8192, variant=256)["block_n"] == 256 and c(512, 512, 512, variant=512)["block_n"] == 512
    assert c(1536, 2304, 65536, variant=256, split_k=0)["split_k"] == 4      # the automatic K split
    assert c(8192, 8192, 8192, tf32=True)["block_n"] == 512
    assert c(8192, 8192, 8192, sm_count=132)["block_n"] in (256, 512)        # another SM count: still a valid answer
    try:
        sp.tune(wide=1)
        assert c(8192, 8192, 8192)["block_n"] == 256
    finally:
        sp.tune()


def test_tile_narrows_when_256_wide_tiles_underfill_the_machine(sp):
    c = sp.choice
    assert c(768, 3072, 3072)["block_n"] == 128        # 36 tiles of 256 columns for 74 CTA pairs; 72 of 128
    assert c(1536, 768, 65536)["block_n"] == 64        # 18 -> 72 tiles
    assert c(768, 2816, 65536)["block_n"] == 128       # 33 -> 66 tiles, still one wave
    assert c(2304, 2816, 65536)["block_n"] == 256      # 99 tiles = two waves; 198 narrower ones = three waves that
                                                       # are not short enough (narrow tiles are bound by L2)
    assert c(2048, 2048, 2048)["block_n"] == 256       # 64 tiles: narrower tiles would need a second wave
    assert c(12288, 24576, 1536)["block_n"] == 256     # many waves: nothing to gain
    try:
        sp.tune(keep_wide_tiles=True)
        assert c(768, 3072, 3072)["block_n"] == 256
    finally:
        sp.tune()


def test_automatic_mode_picks_stream_k_for_a_thin_last_wave(sp):
    """split_k = 0 resolves to stream-K (-1) when several waves of 256-wide tiles end in a wave that is less
    than half full and the modelled gain is at least 7 %; otherwise tiles run whole."""
    assert sp.choice(4096, 4096, 4096, split_k=0)["split_k"] == -1      # 3 waves + 34 of 74
    assert sp.choice(2304, 2816, 65536, split_k=0)["split_k"] == -1     # 1 wave + 25 of 74
    assert sp.choice(8192, 8192, 2048, split_k=0)["split_k"] == 1       # 13 waves + 62 of 74: runs whole
    assert sp.choice(4096, 4096, 1024, split_k=0)["split_k"] == 1       # K too short to pay for the reduce-adds
    assert sp.choice(4096, 4096, 4096, split_k=1)["split_k"] == 1       # the caller asked for whole tiles
    assert sp.choice(4096, 4096, 4096, split_k=0, sm_count=128)["split_k"] == 1  # 256 tiles = 4 full waves of 64


def test_store_bound_problems_run_on_single_ctas(sp):
    """Many tiles and at most four K blocks: the launch is bound by writing C, and single CTAs store faster
    than pairs; from K = 512 on the pair tile stays."""
    c = sp.choice(32768, 65536, 48)
    assert (c["cta_group"], c["block_n"], c["split_k"]) == (1, 256, 1)
    assert sp.choice(16384, 16384, 256)["cta_group"] == 1
    assert sp.choice(16384, 16384, 512)["cta_group"] == 2
    assert sp.choice(2048, 2048, 128)["cta_group"] == 2     # 64 pair tiles: not store-bound, latency-bound
    assert sp.choice(16384, 16384, 128, tf32=True)["cta_group"] == 2   # tf32 has CTA-pair kernels only
