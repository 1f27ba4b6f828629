// Launch-plan arithmetic of the sm_100a GEMM kernels, shared by device code, the host-side launch
// paths, the plan entry points of the C ABI and the host-side model of the barrier protocol: the
// parameter block, the decoding of a CTA group's i-th work item (tile raster, K split, stream-K share)
// and the chunk schedule of the 256 x 512 kernel.  Pure arithmetic: no CUDA call, no memory access.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define SPORK_HD __host__ __device__ __forceinline__
#else
#define SPORK_HD inline
#endif

namespace spork {
namespace gemm_sm100 {

struct Params {
    uint32_t M, N, K;
    uint32_t tiles_m, tiles_n;   // output tiles (tile = kBlockM*CG x BLOCK_N)
    uint32_t split_k;            // >= 1
    uint32_t split_inner;        // 1: the K ranges of one tile are neighbours in the work list (K fastest), 0: K slowest
    uint32_t batches;            // >= 1: independent problems A[l] * B[l]^T -> C[l], contiguous in memory
    uint32_t kb_per_split;       // K blocks per split
    uint32_t num_kb;             // ceil(K / kBlockK)
    uint32_t use_tma_store;      // 0: guarded scalar stores (N % 4 != 0)
    uint32_t stages;             // ring depth in use (<= Config::kStages)
    uint32_t group_m;            // raster: m-tiles per group
    uint32_t l2_hints;           // bit 0: A loads evict_last, bit 1: B loads evict_last, bit 2: B loads evict_first
    uint32_t backoff_ns;         // sleep between polls of the long (epilogue / producer) waits; 0 = spin
    // stream-K: the first `dp_tiles` tiles of the raster (whole waves) run tile by tile; each of the last
    // `sk_tiles` (fewer than there are CTA groups) is cut along K into `sk_extra` ranges of `sk_share` K
    // blocks, one (tile, range) per CTA group, all groups running theirs at the same time over the same K
    // offsets (so concurrent CTAs still share operand strips in L2), and reduce-added into C, which the
    // kernel itself zeroes there at its start.
    uint32_t dp_tiles, sk_tiles;
    uint32_t sk_share, sk_extra; // K blocks per range, ranges per tile
    uint32_t sk_target;          // value of sk_counter[0] from which every share is zeroed: the grid's epilogue warps
    uint32_t wide_skew;          // 256 x 512 tiles: K blocks of one accumulator half issued ahead of the other at both
                                 // ends of a tile (1 .. ring depth)
    uint32_t experiment;         // diagnostics: bit 3 (256 x 512 kernel, results unchanged) = plain stores instead of TMA
                                 // stores.  Results undefined: bit 0 = epilogue drops its stores,
                                 // bit 1 = producer stops issuing loads once the ring has been filled once,
                                 // bit 2 = epilogue stores straight from registers (no shared-memory staging)
    uint32_t trace_items;        // capacity of `trace` in work items
    float* C;
    uint32_t* status;            // device status word
    unsigned long long* trace;   // optional (256 x 512 kernel): SM-clock stamps of CTA 0's tile hand-overs, 8 per work item
    uint32_t* sk_counter;        // [0] counts the warps that have finished zeroing their share of the stream-K tiles,
                                 // [1] the CTAs that have left; the last one to leave zeroes both
};
// The kernels take three 128-byte tensor maps and this block.  Measured: with more than 512 bytes of kernel
// parameters a launch bound by its TMA stores (32768 x 65536 x 48) runs 15 % slower (1.93 ms against 1.67 ms,
// the same code with 8 bytes of padding added here), so the block stays within 128 bytes.
static_assert(sizeof(Params) <= 128, "kernel parameters must stay within 512 bytes");

struct WorkItem {
    uint32_t m_tile, n_tile, kb_begin, kb_end, split, batch;
    bool reduce;  // the partial tile is added into C instead of stored
};

// Grouped raster (the superblock idea of gemm/gemm_sm90.cu:318-345): work items
// that run at the same time cover kGroupM m-tiles by a run of n-tiles; the groups
// alternate their direction along n.
SPORK_HD void decode_tile(const Params& p, uint32_t t, WorkItem& w)
{
    const uint32_t group_size = p.group_m * p.tiles_n;
    const uint32_t g = t / group_size;
    const uint32_t first_m = g * p.group_m;
    const uint32_t gm = (p.tiles_m - first_m) < p.group_m ? (p.tiles_m - first_m) : p.group_m;
    const uint32_t r = t % group_size;
    w.m_tile = first_m + r % gm;
    w.n_tile = r / gm;
    // every other group walks the n-tiles backwards: the B strips the previous group touched last are the
    // first to be used again while they are still in L2 (+0.5 % at 8192^3 with the part at its power cap)
    if (g & 1u) {
        w.n_tile = p.tiles_n - 1u - w.n_tile;
    }
}

// Work of CTA group `g` of `G`.  Without stream-K: items g, g+G, ... of the (split, tile) list.  With
// stream-K: first the whole tiles g, g+G, ... < dp_tiles, then at most one K range of one of the remaining tiles.
SPORK_HD uint32_t group_item_count(const Params& p, uint32_t g, uint32_t G)
{
    if (p.sk_tiles == 0) {
        const uint32_t items = p.tiles_m * p.tiles_n * p.split_k * p.batches;
        return items > g ? (items - g - 1) / G + 1 : 0;
    }
    const uint32_t n1 = p.dp_tiles / G;  // dp_tiles is a multiple of G
    return n1 + (g < p.sk_tiles * p.sk_extra ? 1u : 0u);
}

SPORK_HD WorkItem group_item(const Params& p, uint32_t g, uint32_t G, uint32_t i)
{
    WorkItem w;
    if (p.sk_tiles == 0) {
        const uint32_t item = g + i * G;
        const uint32_t tiles = p.tiles_m * p.tiles_n;
        // Within a batch entry the list is either tile-fastest (every tile's first K range, then every
        // tile's second one: gemm_sm90_k_mode::split_k_outer) or K-fastest (a tile's ranges are neighbours,
        // so they run at the same time on different CTA groups: split_k_inner), gemm/gemm_sm90.cu:1096-1114.
        const uint32_t per_batch = tiles * p.split_k;
        const uint32_t r = item % per_batch;
        w.batch = item / per_batch;
        w.split = p.split_inner ? r % p.split_k : r / tiles;
        decode_tile(p, p.split_inner ? r / p.split_k : r % tiles, w);
        w.kb_begin = w.split * p.kb_per_split;
        const uint32_t e = w.kb_begin + p.kb_per_split;
        w.kb_end = e < p.num_kb ? e : p.num_kb;
        w.reduce = p.split_k > 1;
        return w;
    }
    w.split = 0;
    w.batch = 0;   // stream-K is never planned for a batch
    const uint32_t n1 = p.dp_tiles / G;
    if (i < n1) {
        decode_tile(p, g + i * G, w);
        w.kb_begin = 0;
        w.kb_end = p.num_kb;
        w.reduce = false;
        return w;
    }
    // the group's one stream-K item: ranges of one tile sit sk_tiles groups apart
    w.split = g / p.sk_tiles;
    decode_tile(p, p.dp_tiles + g % p.sk_tiles, w);
    w.kb_begin = w.split * p.sk_share;
    const uint32_t e = w.kb_begin + p.sk_share;
    w.kb_end = e < p.num_kb ? e : p.num_kb;
    w.reduce = true;
    return w;
}

// Sizes of the chunks a tile's K-blocks are issued in.  Inside a chunk the MMAs of H0 come first, then
// those of H1.  The first and the last chunk are `skew` K-blocks long (shorter tiles are cut in two, or
// run as one chunk), the ones between are single K-blocks.  Pure arithmetic, shared with the host-side
// model of the schedule.
SPORK_HD uint32_t wide_chunk(uint32_t n, uint32_t done, uint32_t skew)
{
    const uint32_t rem = n - done;
    if (done == 0) {
        return n >= 2 * skew ? skew : (n > skew ? n - n / 2 : n);
    }
    return rem <= skew ? rem : 1u;
}

// split_k = 0 ("choose"): a problem with fewer output tiles than CTA groups and a long K leaves SMs idle;
// cutting K into s ranges turns it into tiles * s work items.  Pick the s (1..16, at least 8 K blocks per
// range) with the smallest modelled time: waves(s) * (K blocks per range * cycles per block + epilogue),
// where a reduce-add epilogue is dearer than a store.  Only for 256-wide tiles: narrower ones are chosen
// for problems that are bound by memory, where this model does not hold.  Pure arithmetic.
inline uint32_t choose_split(uint32_t M, uint32_t N, uint32_t K, uint32_t tile_m, uint32_t block_n, uint32_t cta_group,
                             uint32_t elems_k, int max_ctas, int sm_count, uint32_t batches)
{
    const uint64_t tiles = (uint64_t)((M + tile_m - 1) / tile_m) * ((N + block_n - 1) / block_n) * (batches ? batches : 1);
    const uint32_t num_kb = (K + elems_k - 1) / elems_k;
    uint32_t groups = (uint32_t)(sm_count / (int)cta_group);
    if (max_ctas > 0 && (uint32_t)max_ctas / cta_group < groups) {
        groups = (uint32_t)max_ctas / cta_group;
    }
    if (block_n != 256 || groups == 0 || tiles >= groups || num_kb < 16) {
        return 1;
    }
    const uint64_t cycles_per_kb = 512, epilogue_store = 4000, epilogue_reduce = 6000;
    uint32_t best = 1;
    uint64_t best_time = (uint64_t)num_kb * cycles_per_kb + epilogue_store;  // one wave, s = 1
    for (uint32_t s = 2; s <= 16; ++s) {
        const uint32_t kb_per = (num_kb + s - 1) / s;
        if (kb_per < 8) {
            break;
        }
        const uint32_t splits = (num_kb + kb_per - 1) / kb_per;  // no empty ranges
        const uint64_t items = tiles * splits;
        const uint64_t waves = (items + groups - 1) / groups;
        const uint64_t t = waves * ((uint64_t)kb_per * cycles_per_kb + epilogue_reduce);
        if (t < best_time) {
            best_time = t;
            best = splits;
        }
    }
    return best;
}

// Host-side launch plan: tile grid, K split, number of CTA groups and the stream-K partition.  Pure
// arithmetic (no CUDA call), shared by the launch paths and by spork_gemm_sm100_plan.
inline void plan_launch(Params& p, uint32_t& groups, uint32_t M, uint32_t N, uint32_t K, uint32_t tile_m,
                        uint32_t block_n, uint32_t cta_group, uint32_t elems_k, uint32_t split_k, bool stream_k,
                        int max_ctas, int sm_count, uint32_t batches = 1)
{
    p.batches = batches < 1 ? 1 : batches;
    if (p.batches > 1) {
        stream_k = false;
    }
    p.M = M;
    p.N = N;
    p.K = K;
    p.tiles_m = (M + tile_m - 1) / tile_m;
    p.tiles_n = (N + block_n - 1) / block_n;
    p.num_kb = (K + elems_k - 1) / elems_k;
    if (split_k > p.num_kb) {
        split_k = p.num_kb;
    }
    if (split_k < 1) {
        split_k = 1;
    }
    p.kb_per_split = (p.num_kb + split_k - 1) / split_k;
    p.split_k = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty splits
    p.use_tma_store = (N % 4 == 0) ? 1u : 0u;
    p.dp_tiles = 0;
    p.sk_tiles = 0;
    p.sk_share = 0;
    p.sk_extra = 0;
    const uint64_t items = (uint64_t)p.tiles_m * p.tiles_n * p.split_k * p.batches;
    groups = (uint32_t)(sm_count / (int)cta_group);
    if (max_ctas > 0 && (uint32_t)max_ctas / cta_group < groups) {
        groups = (uint32_t)max_ctas / cta_group;
    }
    if (groups == 0) {
        groups = 1;
    }
    const uint32_t tiles = p.tiles_m * p.tiles_n;
    const uint32_t tail = tiles % groups;
    // ranges per tail tile: as many as there are groups to run them at once, each at least 4 K blocks long
    uint32_t ranges = tail ? groups / tail : 1;
    uint32_t kb_per_range = p.num_kb;
    if (ranges > 1) {
        kb_per_range = (p.num_kb + ranges - 1) / ranges;
        kb_per_range = kb_per_range < 4 ? 4 : kb_per_range;
        ranges = (p.num_kb + kb_per_range - 1) / kb_per_range;  // no empty ranges
    }
    if (stream_k && p.split_k == 1 && ranges > 1) {
        // whole waves run tile by tile; the tiles of the last partial wave are cut into aligned K ranges
        p.dp_tiles = tiles - tail;
        p.sk_tiles = tail;
        p.sk_share = kb_per_range;
        p.sk_extra = ranges;
        if (p.dp_tiles == 0) {
            groups = tail * ranges;
        }
    } else if (items < groups) {
        groups = (uint32_t)items;
    }
}

}  // namespace gemm_sm100
}  // namespace spork
