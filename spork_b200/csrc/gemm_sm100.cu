// fp16-in / fp32-accumulate GEMM for sm_100a (B200): C[M,N] = A[M,K] . B[N,K]^T.
//
// Takes the place, on Blackwell, of the reference's hand-written Hopper kernel
// (gemm/gemm_sm90.cu: TiledMultiplier, cluster_main_loop, cluster_process_item)
// behind the same launch shape (gemm/gemm_sm90.cu:1344-1360).  The design is
// Blackwell's own rather than a translation:
//
//   * persistent grid, one CTA (or one CTA pair) per SM, static round-robin
//     over output tiles in a grouped raster so that concurrently running CTAs
//     share A row-bands and B column-bands in L2;
//   * warp-specialised: warp 0 = TMA producer, warp 1 = tcgen05.mma issuer
//     (one elected thread) and TMEM owner, warps 2..5 = epilogue;
//   * operands stream through a multi-stage shared-memory ring of 128B-swizzled
//     K-major tiles (64 fp16 = 128 bytes along K per row), filled by unicast
//     TMA loads and handed over with mbarriers (full / empty);
//   * accumulators live in tensor memory, double buffered (2 x block_n columns)
//     so the epilogue of tile i overlaps the main loop of tile i+1;
//   * cta_group::2: a pair of CTAs on neighbouring SMs computes a 256 x block_n
//     tile with one MMA stream issued by the pair's leader.  Each CTA loads its
//     own 128 rows of A and its own half of the B tile with plain unicast loads, and the
//     MMA reads B from both CTAs' shared memory;
//   * epilogue: tcgen05.ld (one thread per accumulator row, 32 columns at a
//     time) -> 128B-swizzled staging slab in shared memory -> TMA store (or TMA
//     reduce-add for split-K).  Ragged edges: TMA zero-fills loads outside the
//     tensors and clips stores.
//
// Every wait is bounded; a wait that runs out sets the device status word and
// the kernel winds down (frees TMEM, returns).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/spork_b200.h"
#include "device_state.h"
#include "gemm_plan.h"
#include "ptx_sm100.cuh"

namespace spork {
namespace gemm_sm100 {

using namespace ptx;

constexpr int kBlockM = 128;        // rows of A (and of the accumulator) per CTA
constexpr int kBlockK = 64;         // fp16 elements along K per stage: one 128-byte swizzle atom
constexpr int kUmmaK = 16;          // K of one tcgen05.mma.kind::f16
// fp32 operands read as tf32 (the reference's own operand type, gemm/gpu_tensor.h:14-16): the same
// 128-byte rows hold 32 elements, one tcgen05.mma.kind::tf32 covers K = 8, so the byte layout of a
// stage, the descriptors and the four MMAs per stage are identical.
constexpr int kBlockKTf32 = 32;
constexpr int kNumThreads = 192;    // 6 warps
constexpr int kEpilogueWarp0 = 2;   // warps 2..5
constexpr int kNumEpilogueWarps = 4;
constexpr int kEpiCols = 32;        // fp32 columns per epilogue chunk = 128 bytes
constexpr int kSlabBytes = 32 * kEpiCols * 4;   // one warp's staging slab: 32 rows x 128 B
constexpr int kSlabsPerWarp = 2;
constexpr int kMaxSmem = 227 * 1024;
constexpr int kGroupM = 8;          // raster: m-tiles per group

// KATOMS: 128-byte column blocks ("atoms", 64 fp16 along K) per stage.  1 is the default; 2 makes every
// TMA request of a row 256 contiguous bytes (two adjacent boxes), which serves skinny, HBM-bound shapes
// better.
template <int CG, int BLOCK_N, int KATOMS = 1>
struct Config {
    static constexpr int kUmmaM = kBlockM * CG;
    static constexpr int kUmmaN = BLOCK_N;
    static constexpr int kBRows = BLOCK_N / CG;  // rows of B this CTA loads per stage
    static constexpr int kAtomABytes = kBlockM * kBlockK * 2;
    static constexpr int kAtomBBytes = kBRows * kBlockK * 2;
    static constexpr int kABytes = KATOMS * kAtomABytes;
    static constexpr int kBBytes = KATOMS * kAtomBBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStagingBytes = kNumEpilogueWarps * kSlabsPerWarp * kSlabBytes;
    static constexpr int kBarrierBytes = 1024;
    static constexpr int kStagesFit = (kMaxSmem - 1024 /*alignment slack*/ - kStagingBytes - kBarrierBytes) / kStageBytes;
    static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
    static constexpr int kAccCols = BLOCK_N;  // TMEM columns of one accumulator buffer
    static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;  // 128 / 256 / 512: powers of two
    static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + kBarrierBytes;
    static_assert(kStages >= 2, "ring too shallow");
    static_assert(kSmemBytes <= kMaxSmem, "shared memory limit");
    static_assert(kUmmaN % 16 == 0 && kUmmaN >= 16 && kUmmaN <= 256, "UMMA N");
};

struct Barriers {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ __forceinline__ void report_timeout(const Params& p, volatile uint32_t* abort_flag, uint32_t role,
                                               uint32_t where)
{
    *abort_flag = 1u;
    // First failure wins; detail = role (bits 24..), barrier kind/index, block id.
    atomicCAS(p.status, 0u, 0x80000000u | (role << 24) | ((where & 0xFFu) << 16) | (blockIdx.x & 0xFFFFu));
}

// kWorkspace = true: each K split stores its partial tile into slab `split` of a
// [split][M][N] fp32 workspace (tmap_c is then a 3-D map over it) instead of
// writing or reduce-adding into C; a second kernel sums the slabs in a fixed order.
// Stream-K tiles are accumulated by reduce-adds, so C must be zero there first.  The epilogue warps have
// nothing to do until the first tile is complete: each zeroes its share of the rows (one tile row at a
// time) and counts itself in; the count is checked before a warp's first reduce-add, whole tiles later.
template <int TILE_M, int TILE_N>
__device__ __forceinline__ void zero_stream_k_tiles(const Params& p, uint32_t warp_index, uint32_t warps_total, uint32_t lane)
{
    const uint32_t rows_total = p.sk_tiles * TILE_M;
    for (uint32_t r = warp_index; r < rows_total; r += warps_total) {
        WorkItem z;
        decode_tile(p, p.dp_tiles + r / TILE_M, z);
        const uint32_t row = z.m_tile * TILE_M + r % TILE_M;
        const uint32_t col0 = z.n_tile * TILE_N;
        if (row >= p.M || col0 >= p.N) {
            continue;
        }
        const uint32_t cols = p.N - col0 < (uint32_t)TILE_N ? p.N - col0 : (uint32_t)TILE_N;
        float* dst = p.C + (size_t)row * p.N + col0;
        if (p.use_tma_store) {
            // N % 4 == 0 and C is 16-byte aligned: so is every tile row
            for (uint32_t c = lane * 4; c < cols; c += 128) {
                *reinterpret_cast<float4*>(dst + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        } else {
            for (uint32_t c = lane; c < cols; c += 32) {
                dst[c] = 0.0f;
            }
        }
    }
    __threadfence();
    __syncwarp();
    if (lane == 0) {
        red_release_gpu_add(p.sk_counter, 1u);
    }
}

template <int CG, int BLOCK_N, bool kWorkspace = false, bool kTf32 = false, int KATOMS = 1, bool kStreamK = false>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_c, const Params p)
{
    using Cfg = Config<CG, BLOCK_N, KATOMS>;
    extern __shared__ uint8_t smem_raw[];

    const uint32_t warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x / 32, 0);  // provably the same in all lanes
    const uint32_t lane = threadIdx.x % 32;
    const uint32_t cta_rank = CG == 2 ? cluster_ctarank() : 0u;
    const bool is_leader = cta_rank == 0;
    const uint32_t group_id = blockIdx.x / CG;       // which CTA pair (or CTA) this is
    const uint32_t num_groups = gridDim.x / CG;

    // Carve shared memory: [ring stages][epilogue slabs][barriers], 1024-byte aligned.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ring_base = smem_base;
    const uint32_t staging_base = ring_base + Cfg::kStages * Cfg::kStageBytes;
    Barriers* bars = reinterpret_cast<Barriers*>(smem_raw + (staging_base + Cfg::kStagingBytes - smem_u32(smem_raw)));
    volatile uint32_t* abort_flag = &bars->abort_flag;

    // Clock probe: CTA 0 notes SM cycles and wall-clock nanoseconds at both ends of the launch; their
    // ratio is the SM clock the kernel really ran at (the power cap moves it far below the nominal clock).
    unsigned long long* probe = reinterpret_cast<unsigned long long*>(p.status + 4);
    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->tmem_full[b]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[b]), kNumEpilogueWarps * CG);
        }
        bars->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
        prefetch_tensormap(&tmap_c);
    }
    if (warp == 1) {
        tmem_alloc<CG>(smem_u32(&bars->tmem_base), Cfg::kTmemCols);
        tmem_relinquish<CG>();
    }
    tcgen05_fence_before();
    __syncthreads();
    if (CG == 2) {
        // The peer's barriers must exist before anything arrives on them remotely.
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    tcgen05_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    // Debug builds test every address and coordinate below against these ranges (see Checker).
    const Checker chk{p.status, smem_base, smem_u32(smem_raw) + (uint32_t)Cfg::kSmemBytes, tmem_base,
                      (uint32_t)Cfg::kTmemCols};
    constexpr uint32_t kOperandBytes = kTf32 ? 4u : 2u;

    // Everything above is independent of earlier work in the stream.  When launched as a programmatic
    // dependent, this CTA may have been set up while the previous kernel was still running on other SMs;
    // from here on it reads and writes global memory, so the previous kernel must be complete.  The next
    // launch may set itself up in the same way while this one runs.
    grid_launch_dependents();
    grid_dependency_wait();
    if (!kWorkspace && blockIdx.x == 0 && threadIdx.x == 0) {
        probe[0] = (unsigned long long)clock64();
        probe[1] = global_timer_ns();
    }

    const uint32_t num_items = group_item_count(p, group_id, num_groups);  // this CTA group's work items
    constexpr int kElemsK = kTf32 ? kBlockKTf32 : kBlockK;  // elements along K per stage

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, issued = 0;
            bool ok = true;
            const uint64_t pol_a = (p.l2_hints & 1u) ? l2_policy_evict_last() : l2_policy_evict_normal();
            const uint64_t pol_b = (p.l2_hints & 2u) ? l2_policy_evict_last()
                                   : (p.l2_hints & 4u) ? l2_policy_evict_first() : l2_policy_evict_normal();
            for (uint32_t item = 0; item < num_items && ok; ++item) {
                const WorkItem w = group_item(p, group_id, num_groups, item);
                const int32_t a_row = (int32_t)(w.m_tile * Cfg::kUmmaM + cta_rank * kBlockM);
                const int32_t b_row = (int32_t)(w.n_tile * BLOCK_N + cta_rank * Cfg::kBRows);
                for (uint32_t kb = w.kb_begin; kb < w.kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag, p.backoff_ns)) {
                        report_timeout(p, abort_flag, 1, stage);
                        ok = false;
                        break;
                    }
                    const uint32_t sa = ring_base + stage * Cfg::kStageBytes;
                    const uint32_t sb = sa + Cfg::kABytes;
                    const uint32_t full = smem_u32(&bars->full[stage]);
                    const bool loads_ok =
                        chk.smem(sa, Cfg::kStageBytes, 1024u, 0x11) &&
                        chk.tma_coords((int32_t)(kb * KATOMS * kElemsK), kOperandBytes, a_row, (int32_t)w.batch, 0x12) &&
                        chk.tma_coords((int32_t)((kb * KATOMS + KATOMS - 1) * kElemsK), kOperandBytes, b_row, 0, 0x13);
                    if (!loads_ok) {
                        ok = false;   // recorded; the other roles end through their bounded waits
                        *abort_flag = 1u;
                        break;
                    }
                    if ((p.experiment & 2u) && issued >= p.stages) {
                        if (is_leader) {
                            mbar_arrive(full);  // hand the stale stage over without loading
                        }
                    } else if (CG == 1) {
                        mbar_arrive_expect_tx(full, Cfg::kStageBytes);
#pragma unroll
                        for (int at = 0; at < KATOMS; ++at) {
                            const int32_t x = (int32_t)((kb * KATOMS + at) * kElemsK);
                            if (p.batches > 1) {   // the maps are 3-D then
                                tma_load_3d_hint(sa + at * Cfg::kAtomABytes, &tmap_a, full, x, a_row, (int32_t)w.batch,
                                                 pol_a);
                                tma_load_3d_hint(sb + at * Cfg::kAtomBBytes, &tmap_b, full, x, b_row, (int32_t)w.batch,
                                                 pol_b);
                            } else {
                                tma_load_2d_hint(sa + at * Cfg::kAtomABytes, &tmap_a, full, x, a_row, pol_a);
                                tma_load_2d_hint(sb + at * Cfg::kAtomBBytes, &tmap_b, full, x, b_row, pol_b);
                            }
                        }
                    } else {
                        // Both CTAs' bytes complete on the leader's barrier.
                        if (is_leader) {
                            mbar_arrive_expect_tx(full, Cfg::kStageBytes * 2);
                        }
                        const uint32_t leader_full = map_to_cta(full, 0);
#pragma unroll
                        for (int at = 0; at < KATOMS; ++at) {
                            const int32_t x = (int32_t)((kb * KATOMS + at) * kElemsK);
                            if (p.batches > 1) {
                                tma_load_3d_pair_hint(sa + at * Cfg::kAtomABytes, &tmap_a, leader_full, x, a_row,
                                                      (int32_t)w.batch, pol_a);
                                tma_load_3d_pair_hint(sb + at * Cfg::kAtomBBytes, &tmap_b, leader_full, x, b_row,
                                                      (int32_t)w.batch, pol_b);
                            } else {
                                tma_load_2d_pair_hint(sa + at * Cfg::kAtomABytes, &tmap_a, leader_full, x, a_row, pol_a);
                                tma_load_2d_pair_hint(sb + at * Cfg::kAtomBBytes, &tmap_b, leader_full, x, b_row, pol_b);
                            }
                        }
                    }
                    ++issued;
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        // The whole warp runs the control flow and one elected lane issues: descriptors, tensor-memory
        // and barrier addresses are then the same in all lanes and can live in uniform registers, which
        // makes an issue a few instructions instead of some sixty cycles from inside a one-lane branch.
        if (is_leader) {
            const bool elected = elect_one();
            constexpr uint32_t idesc = kTf32 ? umma_idesc_tf32_f32(Cfg::kUmmaM, Cfg::kUmmaN)
                                             : umma_idesc_f16_f32(Cfg::kUmmaM, Cfg::kUmmaN);
            uint32_t stage = 0, phase = 0;
            uint32_t local = 0;
            bool ok = true;
            for (uint32_t item = 0; item < num_items && ok; ++item, ++local) {
                const WorkItem w = group_item(p, group_id, num_groups, item);
                const uint32_t buf = local & 1u;
                const uint32_t acc_phase = (local >> 1) & 1u;
                if (!__all_sync(0xFFFFFFFFu, mbar_wait<CG == 2>(smem_u32(&bars->tmem_empty[buf]), acc_phase ^ 1u,
                                                                abort_flag))) {
                    if (elected) {
                        report_timeout(p, abort_flag, 2, 0x40 + buf);
                    }
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * Cfg::kAccCols;
                for (uint32_t kb = w.kb_begin; kb < w.kb_end; ++kb) {
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag))) {
                        if (elected) {
                            report_timeout(p, abort_flag, 2, stage);
                        }
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = ring_base + stage * Cfg::kStageBytes;
                    if (!(chk.smem(sa, Cfg::kStageBytes, 1024u, 0x21) && chk.tmem(tmem_d, Cfg::kAccCols, 0x22))) {
                        *abort_flag = 1u;
                        ok = false;
                        break;
                    }
                    if (elected) {
#pragma unroll
                        for (int at = 0; at < KATOMS; ++at) {
                            const uint64_t desc_a = umma_desc_kmajor_sw128(sa + at * Cfg::kAtomABytes);
                            const uint64_t desc_b = umma_desc_kmajor_sw128(sa + Cfg::kABytes + at * Cfg::kAtomBBytes);
#pragma unroll
                            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                                // 16 fp16 = 32 bytes along K inside the swizzle atom: +2 in the (>>4) address field.
                                const uint32_t acc = (kb != w.kb_begin || at != 0 || k != 0) ? 1u : 0u;
                                if (kTf32) {
                                    umma_tf32_ss<CG>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc, acc);
                                } else {
                                    umma_f16_ss<CG>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc, acc);
                                }
                            }
                        }
                        // Free the stage (in both CTAs) once these MMAs have read it.
                        const uint32_t empty = smem_u32(&bars->empty[stage]);
                        umma_commit<CG>(empty);
                        if (CG == 2) {
                            umma_commit<CG>(map_to_cta(empty, 1));
                        }
                    }
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) {
                    break;
                }
                // Accumulator complete: wake the epilogue warps (of both CTAs).
                const uint32_t tfull = smem_u32(&bars->tmem_full[buf]);
                if (elected) {
                    umma_commit<CG>(tfull);
                    if (CG == 2) {
                        umma_commit<CG>(map_to_cta(tfull, 1));
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t quarter = warp % 4;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
        const uint32_t epi = warp - kEpilogueWarp0;
        const uint32_t slab0 = staging_base + epi * kSlabsPerWarp * kSlabBytes;
        uint32_t local = 0;
        uint32_t slab_sel = 0;
        bool ok = true;
        // kStreamK: the instance stream-K launches run.  The others carry none of its code: measured on a
        // store-bound shape (32768 x 65536 x 48) the epilogue ran 15 % slower with it compiled in, unused.
        bool sk_zeroed = !kStreamK || p.sk_tiles == 0;  // the stream-K tiles are known to be zero everywhere
        if (kStreamK && p.sk_tiles != 0) {
            zero_stream_k_tiles<Cfg::kUmmaM, BLOCK_N>(p, blockIdx.x * kNumEpilogueWarps + epi,
                                                     gridDim.x * kNumEpilogueWarps, lane);
        }
        for (uint32_t item = 0; item < num_items && ok; ++item, ++local) {
            const WorkItem w = group_item(p, group_id, num_groups, item);
            if (kStreamK && w.reduce && !sk_zeroed) {
                if (!counter_wait(p.sk_counter, p.sk_target, abort_flag)) {
                    if (lane == 0) {
                        report_timeout(p, abort_flag, 3, 0x48);
                    }
                    ok = false;
                    break;
                }
                fence_proxy_async_all();
                sk_zeroed = true;
            }
            const uint32_t buf = local & 1u;
            const uint32_t acc_phase = (local >> 1) & 1u;
            if (!mbar_wait(smem_u32(&bars->tmem_full[buf]), acc_phase, abort_flag, p.backoff_ns)) {
                if (lane == 0) {
                    report_timeout(p, abort_flag, 3, 0x40 + buf);
                }
                ok = false;
                break;
            }
            tcgen05_fence_after();
            const uint32_t row0 = w.m_tile * Cfg::kUmmaM + cta_rank * kBlockM + quarter * 32;
            const uint32_t col0 = w.n_tile * BLOCK_N;
            const uint32_t taddr0 = tmem_base + ((quarter * 32u) << 16) + buf * Cfg::kAccCols;
            const bool rows_live = row0 < p.M && w.kb_begin < w.kb_end;
#pragma unroll 1
            for (int c = 0; c < BLOCK_N / kEpiCols; ++c) {
                uint32_t r[32];
                if (!chk.tmem(taddr0 + c * kEpiCols, kEpiCols, 0x31)) {
                    continue;
                }
                tmem_ld_32x32b_x32(taddr0 + c * kEpiCols, r);
                tmem_ld_wait();
                const uint32_t col = col0 + c * kEpiCols;
                if (!rows_live || col >= p.N || (p.experiment & 1u)) {
                    continue;  // warp-uniform
                }
                if (!kWorkspace && (p.experiment & 4u)) {
                    // straight from registers: every thread writes the 128 contiguous bytes of its row
                    const uint32_t row = row0 + lane;
                    if (row < p.M && col + 32 <= p.N) {
                        float4* dst = reinterpret_cast<float4*>(p.C + ((size_t)w.batch * p.M + row) * p.N + col);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                        }
                    }
                    continue;
                }
                if (kWorkspace || p.use_tma_store) {
                    const uint32_t slab = slab0 + slab_sel * kSlabBytes;
                    slab_sel ^= 1u;
                    if (!(chk.smem(slab, kSlabBytes, 1024u, 0x32) &&
                          chk.tma_coords((int32_t)col, 4u, (int32_t)row0, (int32_t)(kWorkspace ? w.split : w.batch), 0x33))) {
                        continue;
                    }
                    // The store issued two chunks ago read this slab; make sure it is done.
                    if (lane == 0) {
                        bulk_wait_group_read<kSlabsPerWarp - 1>();
                    }
                    __syncwarp();
                    // Row `lane` of the slab, 16-byte chunks XOR-swizzled by (row & 7):
                    // the layout a 128B-swizzle tensor map expects, and conflict free.
                    const uint32_t row_addr = slab + lane * 128u;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        st_shared_v4(row_addr + (((uint32_t)j ^ (lane & 7u)) << 4), r[4 * j], r[4 * j + 1],
                                     r[4 * j + 2], r[4 * j + 3]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (kWorkspace) {
                            tma_store_3d(&tmap_c, slab, (int32_t)col, (int32_t)row0, (int32_t)w.split);
                        } else if (p.batches > 1) {
                            if (w.reduce) {
                                tma_reduce_add_3d(&tmap_c, slab, (int32_t)col, (int32_t)row0, (int32_t)w.batch);
                            } else {
                                tma_store_3d(&tmap_c, slab, (int32_t)col, (int32_t)row0, (int32_t)w.batch);
                            }
                        } else if (w.reduce) {
                            tma_reduce_add_2d(&tmap_c, slab, (int32_t)col, (int32_t)row0);
                        } else {
                            tma_store_2d(&tmap_c, slab, (int32_t)col, (int32_t)row0);
                        }
                        bulk_commit_group();
                    }
                } else {
                    const uint32_t row = row0 + lane;
                    if (row < p.M) {
                        float* dst = p.C + ((size_t)w.batch * p.M + row) * p.N + col;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (col + j < p.N) {
                                if (w.reduce) {
                                    atomicAdd(dst + j, __uint_as_float(r[j]));
                                } else {
                                    dst[j] = __uint_as_float(r[j]);
                                }
                            }
                        }
                    }
                }
            }
            // All of this warp's reads of the accumulator buffer are complete.
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                const uint32_t tempty = smem_u32(&bars->tmem_empty[buf]);
                if (CG == 1) {
                    mbar_arrive(tempty);
                } else {
                    mbar_arrive_cluster(map_to_cta(tempty, 0));
                }
            }
        }
        if (lane == 0) {
            // shared memory must outlive the stores' reads of it; their writes are complete when the kernel is
            bulk_wait_group_read<0>();
        }
    }

    // ------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    if (CG == 2) {
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<CG>(tmem_base, Cfg::kTmemCols);
    }
    if (!kWorkspace && blockIdx.x == 0 && threadIdx.x == 0) {
        probe[2] = (unsigned long long)clock64();
        probe[3] = global_timer_ns();
    }
    if (kStreamK && p.sk_tiles != 0 && threadIdx.x == 0) {
        // The last CTA to leave puts the launch's two counters back to zero (every CTA is past its check of
        // the first one by now), so the next launch that is handed them starts from zero whatever it is:
        // the value a launch waits for is then a property of its grid, not of the launches before it.
        __threadfence();
        if (atomicAdd(p.sk_counter + 1, 1u) == gridDim.x - 1u) {
            p.sk_counter[0] = 0u;
            p.sk_counter[1] = 0u;
            __threadfence();
        }
    }
}

}  // namespace gemm_sm100
}  // namespace spork

#include "gemm_sm100_wide.cuh"

namespace spork {
namespace gemm_sm100 {

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        }
    });
    return fn;
}

// Encoded tensor maps are remembered per host thread, keyed by everything that goes into the encoding
// (base address, extents, box, element type): a launch on operands seen before costs no driver call
// (the reference encodes three maps on every launch, gemm/gemm_sm90.cu:1167-1206, about a microsecond
// each).  A map describes addresses and shapes only, never contents, so an entry cannot go stale: memory
// freed and allocated again at the same address with the same shape is described by the same map.
struct TmapKey {
    const void* base;
    uint64_t rows, cols, batches;
    uint32_t box_rows, box_cols, dtype, dims;
    bool operator==(const TmapKey& o) const
    {
        return base == o.base && rows == o.rows && cols == o.cols && batches == o.batches && box_rows == o.box_rows &&
               box_cols == o.box_cols && dtype == o.dtype && dims == o.dims;
    }
};

struct TmapCache {
    static constexpr int kSlots = 32;  // searched linearly; replaced round-robin
    struct Slot {
        bool valid = false;
        TmapKey key{};
        CUtensorMap map;
    };
    Slot slots[kSlots];
    int next = 0;
};
static thread_local TmapCache t_tmap_cache;
static std::atomic<uint64_t> g_tmap_hits{0}, g_tmap_misses{0};

static bool tmap_lookup(const TmapKey& key, CUtensorMap* map)
{
    for (const TmapCache::Slot& s : t_tmap_cache.slots) {
        if (s.valid && s.key == key) {
            *map = s.map;
            g_tmap_hits.fetch_add(1, std::memory_order_relaxed);
            return true;
        }
    }
    g_tmap_misses.fetch_add(1, std::memory_order_relaxed);
    return false;
}

static void tmap_remember(const TmapKey& key, const CUtensorMap& map)
{
    TmapCache& c = t_tmap_cache;
    TmapCache::Slot& s = c.slots[c.next];
    c.next = (c.next + 1) % TmapCache::kSlots;
    s.valid = true;
    s.key = key;
    s.map = map;
}

// 2-D row-major tensor map: `cols` is the contiguous dimension.
static int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                        uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols)
{
    const TmapKey key{base, rows, cols, 1, box_rows, box_cols, (uint32_t)dtype, 2};
    if (tmap_lookup(key, map)) {
        return 0;
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        return SPORK_ERR_DRIVER;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * elem_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return SPORK_ERR_DRIVER;
    }
    tmap_remember(key, *map);
    return 0;
}

// 3-D map over `batches` such matrices stored one after the other; a box never spans two of them, so
// ragged rows are zero-filled (loads) or clipped (stores) per matrix.
static int make_tmap_3d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                        uint64_t batches, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols)
{
    const TmapKey key{base, rows, cols, batches, box_rows, box_cols, (uint32_t)dtype, 3};
    if (tmap_lookup(key, map)) {
        return 0;
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        return SPORK_ERR_DRIVER;
    }
    const cuuint64_t dims[3] = {cols, rows, batches};
    const cuuint64_t strides[2] = {cols * elem_bytes, rows * cols * elem_bytes};
    const cuuint32_t box[3] = {box_cols, box_rows, 1};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    const CUresult r = fn(map, dtype, 3, const_cast<void*>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return SPORK_ERR_DRIVER;
    }
    tmap_remember(key, *map);
    return 0;
}

// Process-wide tuning knobs (spork_gemm_sm100_tune); the defaults are the measured best.
struct Tuning {
    int stages = 0;       // 0 = as deep as shared memory allows
    int group_m = 8;
    int l2_hints = 0;
    int backoff_ns = 0;
    int experiment = 0;
    int k_atoms = 0;      // 0 = choose; 1 / 2 = 128-byte column blocks per stage
    int wide = 0;         // 256 x 512 tiles: 0 = choose, 1 = never, 2 = whenever the shape allows
    int wide_skew = 0;    // 0 = default (ring depth)
    int wide_group_m = 0; // 0 = default raster group of the 256 x 512 kernel
    int no_early_launch = 0;  // 1: launches are not programmatic dependents (no overlap with the previous kernel's tail)
    int narrow = 0;           // 1: problems that underfill the machine keep 256-wide tiles (no 128- / 64-wide choice)
    unsigned long long* trace = nullptr;  // spork_gemm_sm100_trace
    uint32_t trace_items = 0;
};
static Tuning g_tuning;

// Operand loads carry an L2 evict-last hint unless told otherwise: strips of A and B are read again by
// later tiles and waves, and keeping them in L2 saves DRAM reads, i.e. power, i.e. clock.  Measured on a
// part held at its power cap (300 launches per sample, alternated): 8192^3 1203 against 1184 TFLOP/s,
// 4096^3 1103 against 1079, 2048^3 909 against 863, 32768 x 40016 x 816 844 against 772; never slower.
// Tuning value 0 = this default, 1 / 2 / 3 = A / B / both evict-last, 4 = B evict-first, 8 = no hints.
static uint32_t effective_l2_hints(int tuned)
{
    const uint32_t h = (uint32_t)tuned & 15u;
    if (h == 0) {
        return 3u;
    }
    return (h & 8u) ? 0u : h;
}

template <int CG, int BLOCK_N, bool kTf32 = false, int KATOMS = 1>
static int launch(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C, uint32_t split_k,
                  int max_ctas, DeviceState& dev, cudaStream_t stream, bool stream_k = false, uint32_t batches = 1,
                  bool split_inner = false)
{
    using Cfg = Config<CG, BLOCK_N, KATOMS>;
    // stream-K has instances of its own (not for every ring-stage variant: a request without one runs whole)
    constexpr bool kHasStreamK = KATOMS == 1;
    stream_k = stream_k && kHasStreamK;
    auto kernel = gemm_kernel<CG, BLOCK_N, false, kTf32, KATOMS>;
    auto kernel_sk = gemm_kernel<CG, BLOCK_N, false, kTf32, KATOMS, kHasStreamK>;
    constexpr int kElemsK = kTf32 ? kBlockKTf32 : kBlockK;
    constexpr CUtensorMapDataType kOperandType = kTf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    constexpr uint32_t kOperandBytes = kTf32 ? 4 : 2;

    static std::once_flag attr_once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(attr_once[dev.ordinal], [&] {
        attr_err[dev.ordinal] =
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (kHasStreamK && attr_err[dev.ordinal] == cudaSuccess) {
            attr_err[dev.ordinal] =
                cudaFuncSetAttribute(kernel_sk, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        }
    });
    if (attr_err[dev.ordinal] != cudaSuccess) {
        return (int)attr_err[dev.ordinal];
    }

    Params p{};
    uint32_t groups = 1;
    plan_launch(p, groups, M, N, K, Cfg::kUmmaM, BLOCK_N, CG, kElemsK * KATOMS, split_k, stream_k, max_ctas,
                dev.sm_count, batches);
    p.split_inner = split_inner ? 1u : 0u;
    p.C = C;
    p.status = dev.status_word;
    const Tuning tune = g_tuning;
    p.stages = (tune.stages >= 2 && tune.stages <= Cfg::kStages) ? (uint32_t)tune.stages : (uint32_t)Cfg::kStages;
    p.group_m = tune.group_m >= 1 ? (uint32_t)tune.group_m : (uint32_t)kGroupM;
    p.l2_hints = effective_l2_hints(tune.l2_hints);
    p.backoff_ns = (uint32_t)tune.backoff_ns;
    p.experiment = (uint32_t)tune.experiment;

    CUtensorMap tmap_a, tmap_b, tmap_c;
    int rc = p.batches > 1 ? make_tmap_3d(&tmap_a, kOperandType, kOperandBytes, A, p.batches, M, K, kBlockM, kElemsK)
                           : make_tmap_2d(&tmap_a, kOperandType, kOperandBytes, A, M, K, kBlockM, kElemsK);
    if (rc) {
        return rc;
    }
    rc = p.batches > 1 ? make_tmap_3d(&tmap_b, kOperandType, kOperandBytes, B, p.batches, N, K, Cfg::kBRows, kElemsK)
                       : make_tmap_2d(&tmap_b, kOperandType, kOperandBytes, B, N, K, Cfg::kBRows, kElemsK);
    if (rc) {
        return rc;
    }
    if (p.use_tma_store) {
        rc = p.batches > 1
                 ? make_tmap_3d(&tmap_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, C, p.batches, M, N, 32, kEpiCols)
                 : make_tmap_2d(&tmap_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, C, M, N, 32, kEpiCols);
        if (rc) {
            return rc;
        }
    } else {
        tmap_c = tmap_a;  // never dereferenced
    }

    if (p.split_k > 1) {
        const cudaError_t e = cudaMemsetAsync(C, 0, sizeof(float) * (size_t)M * N * p.batches, stream);
        if (e != cudaSuccess) {
            return (int)e;
        }
    }

    if (p.sk_tiles != 0) {
        // the kernel zeroes the stream-K tiles itself; its CTAs meet at one of the device's counter pairs
        p.sk_counter = reserve_sk_counter(dev);
        p.sk_target = groups * CG * kNumEpilogueWarps;
    }

    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(groups * CG, 1, 1);
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // the kernel sets itself up before it waits for the previous kernel in the stream (see grid_dependency_wait)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tune.no_early_launch ? 1 : 2;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, p.sk_tiles != 0 ? kernel_sk : kernel, tmap_a, tmap_b, tmap_c, p);
    return (int)e;
}

// The 256 x 512 kernel: same plan, maps and status word as launch<2, ...>.
template <bool kTf32>
static int launch_wide(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C, uint32_t split_k,
                       int max_ctas, DeviceState& dev, cudaStream_t stream, bool split_inner = false)
{
    using Cfg = WideConfig;
    auto kernel = gemm_wide_kernel<kTf32>;
    constexpr int kElemsK = kTf32 ? kBlockKTf32 : kBlockK;
    constexpr CUtensorMapDataType kOperandType = kTf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    constexpr uint32_t kOperandBytes = kTf32 ? 4 : 2;

    static std::once_flag attr_once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(attr_once[dev.ordinal], [&] {
        attr_err[dev.ordinal] =
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    });
    if (attr_err[dev.ordinal] != cudaSuccess) {
        return (int)attr_err[dev.ordinal];
    }

    Params p{};
    uint32_t groups = 1;
    plan_launch(p, groups, M, N, K, 2 * kBlockM, kWideN, 2, kElemsK, split_k, false, max_ctas, dev.sm_count, 1);
    p.split_inner = split_inner ? 1u : 0u;
    p.C = C;
    p.status = dev.status_word;
    const Tuning tune = g_tuning;
    p.stages = (uint32_t)kWideStages;
    p.group_m = tune.wide_group_m >= 1 ? (uint32_t)tune.wide_group_m : (uint32_t)kWideGroupM;
    p.l2_hints = effective_l2_hints(tune.l2_hints);
    p.backoff_ns = (uint32_t)tune.backoff_ns;
    p.experiment = (uint32_t)tune.experiment & 9u;
    p.wide_skew = tune.wide_skew >= 1 ? (uint32_t)tune.wide_skew : (uint32_t)kWideStages;
    p.trace = tune.trace;
    p.trace_items = tune.trace_items;

    CUtensorMap tmap_a, tmap_b, tmap_c;
    int rc = make_tmap_2d(&tmap_a, kOperandType, kOperandBytes, A, M, K, kBlockM, kElemsK);
    if (rc) {
        return rc;
    }
    rc = make_tmap_2d(&tmap_b, kOperandType, kOperandBytes, B, N, K, kWideHalfN / 2, kElemsK);
    if (rc) {
        return rc;
    }
    if (p.use_tma_store) {
        rc = make_tmap_2d(&tmap_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, C, M, N, 32, kEpiCols);
        if (rc) {
            return rc;
        }
    } else {
        tmap_c = tmap_a;  // never dereferenced
    }
    if (p.split_k > 1) {
        const cudaError_t e = cudaMemsetAsync(C, 0, sizeof(float) * (size_t)M * N, stream);
        if (e != cudaSuccess) {
            return (int)e;
        }
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(groups * 2, 1, 1);
    cfg.blockDim = dim3(kWideThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tune.no_early_launch ? 1 : 2;
    return (int)cudaLaunchKernelEx(&cfg, kernel, tmap_a, tmap_b, tmap_c, p);
}

static bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// Whether a problem whose tile is left to the library runs with 256 x 512 tiles.  They move a quarter fewer
// operand bytes per FLOP, which is what a compute-bound problem at the power limit is short of, but their
// tiles are twice as coarse: the problem must fill at least two waves of them, waste little of the last
// tile column, and be deep enough for the tile ends to be a small part of a tile.
static bool want_wide_tiles(uint32_t M, uint32_t N, uint32_t K, int max_ctas, int sm_count)
{
    if (g_tuning.wide == 1) {
        return false;
    }
    if (g_tuning.wide == 2) {
        return true;
    }
    uint32_t groups = (uint32_t)sm_count / 2u;
    if (max_ctas > 0 && (uint32_t)max_ctas / 2u < groups) {
        groups = (uint32_t)max_ctas / 2u;
    }
    const uint64_t tiles_n = (N + kWideN - 1) / kWideN;
    const uint64_t tiles = (uint64_t)((M + 255) / 256) * tiles_n;
    const uint64_t padded_n = tiles_n * kWideN;
    // The coarser tiles must not cost a wave: 15360 x 1536 x 8192 is 180 wide tiles = 2.4 waves of 74 pairs
    // (three waves, 81 % of the machine-time used) but 360 narrow ones = 4.9 waves (97 %).  Compare the
    // work in units of narrow tiles per wave slot and allow the wide tile a 2 % worse fill.
    if (groups > 0) {
        const uint64_t narrow_tiles = (uint64_t)((M + 255) / 256) * ((N + 255) / 256);
        const uint64_t wide_slots = (tiles + groups - 1) / groups * groups * 2;         // in narrow-tile units
        const uint64_t narrow_slots = (narrow_tiles + groups - 1) / groups * groups;
        if (wide_slots * 100 > narrow_slots * 102) {
            return false;
        }
    }
    // K: the tile ends cost about 5000 cycles of tensor-pipe idle time (the epilogue cannot hide behind a
    // second accumulator), against 1024 cycles per K block; measured at the power limit the wide tile wins
    // from K = 4096 upwards (8192^3 +6 %, 40016 x 32768 x 6400 +3 %) and loses below (8192 x 8192 x 2048 -6 %).
    return groups > 0 && tiles >= 2ull * groups && K >= 4096 && (padded_n - N) * 16 <= N;
}

// What a launch resolves to: tile width (512 = the 256 x 512 kernel), CTAs per tile, 128-byte column
// blocks per ring stage, K split (-1 = stream-K).  Pure arithmetic over the arguments, the SM count and
// the tuning knobs; shared by the launch path and spork_gemm_sm100_choice.
struct TileChoice {
    int block_n, cta_group, k_atoms, split_k;
};

static bool choose_tile(TileChoice& c, uint32_t M, uint32_t N, uint32_t K, int block_n, int cta_group, int split_k,
                        int max_ctas, int sm_count, bool tf32, uint32_t batches)
{
    const bool tile_left_to_library = cta_group == 0;
    const bool split_left_to_library = split_k == 0;
    if (block_n == kWideN) {
        // 256 x 512 tiles on request: CTA pairs only, one matrix, output-stationary or split-K
        if ((cta_group != 0 && cta_group != 2) || batches != 1 || split_k < 0) {
            return false;
        }
        c = TileChoice{kWideN, 2, 1, split_k == 0 ? 1 : split_k};
        return true;
    }
    if (cta_group == 0) {
        // The caller left the tile to the library.  A problem that fills a small part of one wave and
        // has a short K is bound by latencies, not by throughput: a single CTA per tile starts 1.5-2 us
        // sooner than a pair (no cluster to form) and 128-wide tiles spread the work over more SMs
        // (160 x 480 x 816: 9.2 us against 12.4 us; 768 x 768 x 32: 6.6 against 8.9).
        cta_group = SPORK_DEFAULT_CTA_GROUP;
        const uint64_t pair_tiles =
            (uint64_t)((M + 255) / 256) * ((N + (uint32_t)block_n - 1) / (uint32_t)block_n) * batches;
        if (!tf32 && split_k == 1 && K <= 1024 && pair_tiles * 4 <= (uint64_t)sm_count) {
            cta_group = 1;
            block_n = block_n > 128 ? 128 : block_n;
        } else if (!tf32 && split_k <= 1 && K <= 256 && pair_tiles >= (uint64_t)sm_count) {
            // A large problem with at most four K blocks per tile is bound by writing C.  Single CTAs then
            // store faster than pairs, whose epilogues wait for each other at every tile (16384 x 16384 x K,
            // GB/s of C written: K = 64 5460 against 5050, 128 5720 / 5060, 256 5550 / 4690; K = 512 equal;
            // from K = 816 on the pair's halved operand traffic wins, 2870 against 2350).
            cta_group = 1;
        }
    }
    if (split_k == 0) {
        split_k = (int)choose_split(M, N, K, 128u * (uint32_t)cta_group, (uint32_t)block_n, (uint32_t)cta_group,
                                    tf32 ? 32u : 64u, max_ctas, sm_count, batches);
    }
    if (tile_left_to_library && cta_group == 2 && block_n == 256 && split_k == 1 && g_tuning.narrow != 1) {
        // A problem with fewer 256-wide tiles than CTA pairs leaves SMs idle; 128- or 64-wide tiles fill the
        // machine instead (768 x 3072 x 3072: 36 tiles of 256 columns, 72 of 128).  Modelled time = waves x
        // (K blocks x cycles per K block + a tile's fixed cost); cycles per K block 550 / 410 / 340 for 256 /
        // 128 / 64 columns: narrower tiles pull more operand bytes per FLOP through L2 (32 / 24 / 20 KB per CTA
        // and K block), and about 60 bytes per clock and SM is what L2 delivers when every SM asks (measured:
        // 2304 x 2816 x 65536 runs 565 cycles per K block with 256-wide and 420 with 128-wide tiles).  The
        // narrower tile must win by 15 %.
        uint32_t groups = (uint32_t)sm_count / 2u;
        if (max_ctas > 0 && (uint32_t)max_ctas / 2u < groups) {
            groups = (uint32_t)max_ctas / 2u;
        }
        if (groups > 0) {
            const uint64_t num_kb = (K + (tf32 ? 32u : 64u) - 1) / (tf32 ? 32u : 64u);
            const uint64_t tiles_m = (uint64_t)((M + 255) / 256) * batches;
            auto cost = [&](uint32_t bn, uint64_t cycles_per_kb) {
                const uint64_t tiles = tiles_m * ((N + bn - 1) / bn);
                return ((tiles + groups - 1) / groups) * (num_kb * cycles_per_kb + 3000);
            };
            const uint64_t c256 = cost(256, 550), c128 = cost(128, 410), c64 = cost(64, 340);
            if (c128 * 100 < c256 * 85 && c128 <= c64) {
                block_n = 128;
            } else if (c64 * 100 < c256 * 85 && c64 < c128) {
                block_n = 64;
            }
        }
    }
    if (tile_left_to_library && cta_group == 2 && block_n == 256 && batches == 1 && split_k == 1 &&
        want_wide_tiles(M, N, K, max_ctas, sm_count)) {
        c = TileChoice{kWideN, 2, 1, 1};
        return true;
    }
    if (split_left_to_library && split_k == 1 && cta_group == 2 && block_n == 256 && batches == 1) {
        // More than one wave of tiles, the last one less than half full: stream-K cuts the tiles of that
        // wave into two or more K ranges that run at the same time (4096^3: 256 tiles = 3 waves of 74 CTA
        // pairs + 34 tiles, each cut in two: 3.5 tile-times instead of 4).  Modelled as in the narrowing
        // above, with a reduce-add epilogue at 6000 cycles; stream-K must win by 7 %.
        Params sp{};
        uint32_t sg = 0;
        plan_launch(sp, sg, M, N, K, 256u, 256u, 2u, tf32 ? 32u : 64u, 1u, true, max_ctas, sm_count, 1);
        if (sp.sk_tiles != 0 && sp.dp_tiles != 0) {
            const uint64_t tile_time = (uint64_t)sp.num_kb * 550 + 3000;
            const uint64_t t_whole = (uint64_t)(sp.dp_tiles / sg + 1) * tile_time;
            const uint64_t t_stream = (uint64_t)(sp.dp_tiles / sg) * tile_time + (uint64_t)sp.sk_share * 550 + 6000;
            if (t_stream * 100 < t_whole * 93) {
                split_k = -1;
            }
        }
    }
    // Two column blocks per stage for skinny problems (few output tiles, long K): their time goes into
    // streaming A from HBM, and 256-byte row segments use the DRAM pages better than 128-byte ones.
    const uint64_t out_tiles =
        (uint64_t)((M + 255) / 256) * ((N + (uint32_t)block_n - 1) / (uint32_t)block_n) * batches;
    const bool wide_k = !tf32 && (g_tuning.k_atoms == 2 ||
                                  (cta_group == 2 && g_tuning.k_atoms == 0 && block_n <= 128 &&
                                   out_tiles <= (uint64_t)sm_count / 2 && K >= 2048));
    c = TileChoice{block_n, cta_group, wide_k ? 2 : 1, split_k};
    return true;
}

static int dispatch(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C, int block_n,
                    int cta_group, int split_k, int max_ctas, cudaStream_t stream, bool tf32 = false,
                    uint32_t batches = 1)
{
    if (tf32 ? (K % 4 != 0) : !spork_gemm_sm100_supports(M, N, K)) {
        return SPORK_ERR_UNSUPPORTED_SHAPE;
    }
    if (M == 0 || N == 0 || batches == 0) {
        return 0;
    }
    // split_k <= -2: |split_k| K ranges, K fastest in the work list (gemm_sm90_k_mode::split_k_inner)
    const bool split_inner = split_k <= -2;
    if (split_inner) {
        split_k = -split_k;
    }
    if (batches > 1 && (split_k == -1 || (uint64_t)batches * ((M + 127) / 128) * ((N + 63) / 64) > 0x3FFFFFFFull)) {
        return SPORK_ERR_BAD_ARGUMENT;  // no stream-K over a batch; the item index is 32 bits wide
    }
    if (!A || !B || !C || !aligned16(A) || !aligned16(B) || !aligned16(C)) {
        // K == 0 with null A/B is still an error only if they would be read; be strict and simple.
        if (!(K == 0 && C && aligned16(C))) {
            return SPORK_ERR_BAD_ARGUMENT;
        }
    }
    if (split_k < -1 || max_ctas < 0) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    if (K == 0) {
        return (int)cudaMemsetAsync(C, 0, sizeof(float) * (size_t)M * N * batches, stream);
    }
    DeviceState* dev = nullptr;
    const int rc = current_device_state(&dev);
    if (rc) {
        return rc;
    }
    TileChoice choice;
    if (!choose_tile(choice, M, N, K, block_n, cta_group, split_k, max_ctas, dev->sm_count, tf32, batches)) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    block_n = choice.block_n;
    cta_group = choice.cta_group;
    const bool stream_k = choice.split_k == -1;
    const uint32_t sk = stream_k ? 1u : (uint32_t)choice.split_k;
    if (choice.block_n == kWideN) {
        return tf32 ? launch_wide<true>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, split_inner)
                    : launch_wide<false>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, split_inner);
    }
    const bool wide_k = choice.k_atoms == 2;
    if (!tf32 && g_tuning.k_atoms == 3 && cta_group == 2 && block_n <= 128) {
        // four column blocks (512 contiguous bytes per row and request): an experiment for the skinny shapes
        return block_n == 64 ? launch<2, 64, false, 4>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner)
                             : launch<2, 128, false, 4>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
    }
    if (wide_k && cta_group == 2) {
        switch (block_n) {
        case 64: return launch<2, 64, false, 2>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        case 128: return launch<2, 128, false, 2>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        case 256: return launch<2, 256, false, 2>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        default: return SPORK_ERR_BAD_ARGUMENT;
        }
    }
    if (wide_k && cta_group == 1) {
        switch (block_n) {
        case 64: return launch<1, 64, false, 2>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        case 128: return launch<1, 128, false, 2>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        case 256: return launch<1, 256, false, 2>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        default: return SPORK_ERR_BAD_ARGUMENT;
        }
    }
#define SPORK_GEMM_CASE(CG_, BN_)                                                               \
    if (cta_group == CG_ && block_n == BN_) {                                                   \
        return launch<CG_, BN_>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);        \
    }
    if (tf32) {
        if (cta_group != 2) {
            return SPORK_ERR_BAD_ARGUMENT;
        }
        switch (block_n) {
        case 64: return launch<2, 64, true>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        case 128: return launch<2, 128, true>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        case 256: return launch<2, 256, true>(M, N, K, A, B, C, sk, max_ctas, *dev, stream, stream_k, batches, split_inner);
        default: return SPORK_ERR_BAD_ARGUMENT;
        }
    }
    SPORK_GEMM_CASE(1, 64)
    SPORK_GEMM_CASE(1, 128)
    SPORK_GEMM_CASE(1, 256)
    SPORK_GEMM_CASE(2, 64)
    SPORK_GEMM_CASE(2, 128)
    SPORK_GEMM_CASE(2, 256)
#undef SPORK_GEMM_CASE
    return SPORK_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------
// Allocation-free variant: deterministic split-K through a workspace that lives
// in a fixed device array of this module instead of allocated memory.
//
// Layout of the array: bytes [0, 256) hold the device status word of this
// variant, bytes [256, 256 + kStaticWorkspaceBytes) the [split][M][ceil4(N)] fp32
// partial products.  Every GPU that loads the library carries the array until
// the process exits.

constexpr size_t kStaticWorkspaceBytes = 64ull << 20;
static __device__ __align__(256) unsigned char g_static_scratch[256 + kStaticWorkspaceBytes];

// C[m][n] = sum over slabs, in ascending slab order, of ws[slab][m][n] (row pitch `pitch` floats).
__global__ void __launch_bounds__(256) reduce_slabs_kernel(const float* ws, float* C, uint32_t M, uint32_t N,
                                                          uint32_t pitch, uint32_t slabs)
{
    const size_t total = (size_t)M * N;
    const size_t slab_stride = (size_t)M * pitch;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t m = (uint32_t)(i / N), n = (uint32_t)(i % N);
        const float* src = ws + (size_t)m * pitch + n;
        float acc = src[0];
        for (uint32_t s = 1; s < slabs; ++s) {
            acc += src[s * slab_stride];
        }
        C[i] = acc;
    }
}

struct StaticDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
};
static StaticDevice g_static_dev[kMaxDevices];
static std::mutex g_static_mutex;

template <int BLOCK_N>
static int launch_static(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C, uint32_t split_k,
                         const StaticDevice& dev, int ordinal, cudaStream_t stream)
{
    constexpr int CG = 2;
    using Cfg = Config<CG, BLOCK_N>;
    auto kernel = gemm_kernel<CG, BLOCK_N, true>;
    static std::once_flag attr_once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(attr_once[ordinal], [&] {
        attr_err[ordinal] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    });
    if (attr_err[ordinal] != cudaSuccess) {
        return (int)attr_err[ordinal];
    }
    Params p{};
    p.batches = 1;
    p.M = M;
    p.N = N;
    p.K = K;
    p.tiles_m = (M + Cfg::kUmmaM - 1) / Cfg::kUmmaM;
    p.tiles_n = (N + BLOCK_N - 1) / BLOCK_N;
    p.num_kb = (K + kBlockK - 1) / kBlockK;
    if (split_k > p.num_kb) {
        split_k = p.num_kb;
    }
    p.kb_per_split = (p.num_kb + split_k - 1) / split_k;
    p.split_k = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
    p.use_tma_store = 1;
    p.C = C;
    p.status = reinterpret_cast<uint32_t*>(dev.scratch);
    p.stages = (uint32_t)Cfg::kStages;
    p.group_m = (uint32_t)kGroupM;
    p.l2_hints = effective_l2_hints(g_tuning.l2_hints);
    p.backoff_ns = 0;
    p.experiment = 0;

    const uint32_t pitch = (N + 3u) & ~3u;  // rows of the workspace are multiples of 16 bytes
    if ((size_t)p.split_k * M * pitch * sizeof(float) > kStaticWorkspaceBytes) {
        return SPORK_ERR_TOO_LARGE;
    }
    float* ws = reinterpret_cast<float*>(dev.scratch + 256);

    CUtensorMap tmap_a, tmap_b, tmap_ws;
    int rc = make_tmap_2d(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, A, M, K, kBlockM, kBlockK);
    if (rc) {
        return rc;
    }
    rc = make_tmap_2d(&tmap_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, B, N, K, Cfg::kBRows, kBlockK);
    if (rc) {
        return rc;
    }
    {
        EncodeTiledFn fn = encode_tiled_fn();
        if (!fn) {
            return SPORK_ERR_DRIVER;
        }
        const cuuint64_t dims[3] = {N, M, p.split_k};
        const cuuint64_t strides[2] = {(cuuint64_t)pitch * 4, (cuuint64_t)M * pitch * 4};
        const cuuint32_t box[3] = {kEpiCols, 32, 1};
        const cuuint32_t elem_strides[3] = {1, 1, 1};
        if (fn(&tmap_ws, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ws, dims, strides, box, elem_strides,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            return SPORK_ERR_DRIVER;
        }
    }
    const uint64_t items = (uint64_t)p.tiles_m * p.tiles_n * p.split_k;
    uint32_t groups = (uint32_t)(dev.sm_count / CG);
    if (groups == 0) {
        groups = 1;
    }
    if (items < groups) {
        groups = (uint32_t)items;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(groups * CG, 1, 1);
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmap_a, tmap_b, tmap_ws, p);
    if (e != cudaSuccess) {
        return (int)e;
    }
    const size_t total = (size_t)M * N;
    const unsigned blocks = (unsigned)((total + 255) / 256 < (size_t)dev.sm_count * 8 ? (total + 255) / 256
                                                                                         : (size_t)dev.sm_count * 8);
    reduce_slabs_kernel<<<blocks, 256, 0, stream>>>(ws, C, M, N, pitch, p.split_k);
    return (int)cudaGetLastError();
}

}  // namespace gemm_sm100
}  // namespace spork

// For callers that must not allocate device memory when they call into this
// library - code running inside a memory arena that already owns the whole GPU,
// a process whose device allocator is locked down after start-up, a latency
// path where cudaMalloc's implicit synchronisation is not acceptable.  The
// other GEMM entry points allocate a status word on a device's first call;
// this one touches only a fixed array that is part of the library image.
//
// Computes the same product as spork_gemm_sm100_f16f32 with K cut into
// `split_k` ranges (>= 1) whose partial products are summed in a fixed order,
// so the result is bit-reproducible for a given split_k.
//
// Limits and rules:
//   * split_k * M * ceil4(N) * 4 bytes must fit the 64 MiB workspace, otherwise
//     SPORK_ERR_TOO_LARGE is returned and nothing is launched;
//   * the first call on each device looks up the array's device address
//     (with that device current) and sets the kernel's shared-memory limit;
//     make that first call before any stream capture starts;
//   * all calls on a device share the one workspace and status word: two calls
//     whose kernels may overlap on the GPU (different streams) race - serialise
//     them; the workspace keeps the last call's partial sums, nothing in it
//     needs to start at zero, the status word is cleared at set-up;
//   * M = N = K = 0 is a query: it synchronises `stream` and returns
//     SPORK_ERR_DEVICE_TIMEOUT (clearing the word) if a kernel launched through
//     this entry point abandoned a bounded wait, else 0.
// It calls no cudaMalloc, cudaFree, or any allocating library routine.
extern "C" int spork_gemm_sm100_f16f32_static(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B,
                                              float* C, int split_k, void* stream_)
{
    using namespace spork::gemm_sm100;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int ordinal = 0;
    cudaError_t e = cudaGetDevice(&ordinal);
    if (e != cudaSuccess) {
        return (int)e;
    }
    if (ordinal < 0 || ordinal >= spork::kMaxDevices) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    StaticDevice dev;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        StaticDevice& d = g_static_dev[ordinal];
        if (!d.ready) {
            int major = 0, sms = 0;
            if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal)) != cudaSuccess ||
                (e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal)) != cudaSuccess) {
                return (int)e;
            }
            if (major != 10) {
                return SPORK_ERR_NO_SM100;
            }
            // In host code `g_static_scratch` is only a handle for the symbol, not a device
            // address: ask the runtime for the address on the current device.
            void* ptr = nullptr;
            if ((e = cudaGetSymbolAddress(&ptr, g_static_scratch)) != cudaSuccess) {
                return (int)e;
            }
            // cleared on the caller's stream and waited for: a blocking memset on the default stream would
            // not be ordered against a stream created as non-blocking
            if ((e = cudaMemsetAsync(ptr, 0, 256, stream)) != cudaSuccess ||
                (e = cudaStreamSynchronize(stream)) != cudaSuccess) {
                return (int)e;
            }
            d.scratch = static_cast<unsigned char*>(ptr);
            d.sm_count = sms;
            d.ready = true;
        }
        dev = d;
    }
    if (M == 0 && N == 0 && K == 0) {  // status query
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) {
            return (int)e;
        }
        uint32_t word = 0;
        if ((e = cudaMemcpyAsync(&word, dev.scratch, sizeof(word), cudaMemcpyDeviceToHost, stream)) != cudaSuccess ||
            (e = cudaStreamSynchronize(stream)) != cudaSuccess) {
            return (int)e;
        }
        if (word != 0) {
            cudaMemsetAsync(dev.scratch, 0, sizeof(word), stream);
            cudaStreamSynchronize(stream);
            return (word >> 28) == 0xCu ? SPORK_ERR_DEVICE_CHECK : SPORK_ERR_DEVICE_TIMEOUT;
        }
        return 0;
    }
    if (!spork_gemm_sm100_supports(M, N, K)) {
        return SPORK_ERR_UNSUPPORTED_SHAPE;
    }
    if (M == 0 || N == 0) {
        return 0;
    }
    if (split_k < 1 || !C || !aligned16(C) || (K != 0 && (!A || !B || !aligned16(A) || !aligned16(B)))) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    if (K == 0) {
        return (int)cudaMemsetAsync(C, 0, sizeof(float) * (size_t)M * N, stream);
    }
    if (N <= 64) {
        return launch_static<64>(M, N, K, A, B, C, (uint32_t)split_k, dev, ordinal, stream);
    }
    if (N <= 128) {
        return launch_static<128>(M, N, K, A, B, C, (uint32_t)split_k, dev, ordinal, stream);
    }
    return launch_static<256>(M, N, K, A, B, C, (uint32_t)split_k, dev, ordinal, stream);
}

// Geometry of a plan as a flat array (see the header for the order).
static bool plan_from_args(spork::gemm_sm100::Params& p, uint32_t& groups, uint32_t M, uint32_t N, uint32_t K,
                           int block_n, int cta_group, int split_k, int max_ctas, int sm_count, int tf32)
{
    if ((block_n != 64 && block_n != 128 && block_n != 256 && block_n != 512) || (cta_group != 1 && cta_group != 2) ||
        (block_n == 512 && (cta_group != 2 || split_k == -1)) || max_ctas < 0 || sm_count < cta_group) {
        return false;
    }
    const bool split_inner = split_k <= -2;
    if (split_inner) {
        split_k = -split_k;
    }
    if (split_k == 0) {
        split_k = (int)spork::gemm_sm100::choose_split(M, N, K, 128u * (uint32_t)cta_group, (uint32_t)block_n,
                                                       (uint32_t)cta_group, tf32 ? 32u : 64u, max_ctas, sm_count, 1);
    }
    spork::gemm_sm100::plan_launch(p, groups, M, N, K, 128u * (uint32_t)cta_group, (uint32_t)block_n,
                                   (uint32_t)cta_group, tf32 ? 32u : 64u, split_k == -1 ? 1u : (uint32_t)split_k,
                                   split_k == -1, max_ctas, sm_count);
    p.split_inner = split_inner ? 1u : 0u;
    p.group_m = (uint32_t)spork::gemm_sm100::kGroupM;
    return true;
}

extern "C" int spork_gemm_sm100_plan(uint32_t M, uint32_t N, uint32_t K, int block_n, int cta_group, int split_k,
                                     int max_ctas, int sm_count, int tf32, uint32_t* out)
{
    spork::gemm_sm100::Params p{};
    uint32_t groups = 0;
    if (!out || !plan_from_args(p, groups, M, N, K, block_n, cta_group, split_k, max_ctas, sm_count, tf32)) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    const uint32_t vals[10] = {p.tiles_m, p.tiles_n, p.num_kb, p.split_k, p.kb_per_split, groups,
                               p.dp_tiles, p.sk_tiles, p.sk_share, p.sk_extra};
    for (int i = 0; i < 10; ++i) {
        out[i] = vals[i];
    }
    return 0;
}

extern "C" int spork_gemm_sm100_plan_items(uint32_t M, uint32_t N, uint32_t K, int block_n, int cta_group,
                                           int split_k, int max_ctas, int sm_count, int tf32, uint32_t group,
                                           uint32_t* out, uint32_t capacity)
{
    spork::gemm_sm100::Params p{};
    uint32_t groups = 0;
    if (!plan_from_args(p, groups, M, N, K, block_n, cta_group, split_k, max_ctas, sm_count, tf32) ||
        group >= groups) {
        return -1;
    }
    const uint32_t count = (M == 0 || N == 0 || K == 0) ? 0u : spork::gemm_sm100::group_item_count(p, group, groups);
    for (uint32_t i = 0; i < count && i < capacity; ++i) {
        const spork::gemm_sm100::WorkItem w = spork::gemm_sm100::group_item(p, group, groups, i);
        out[5 * i + 0] = w.m_tile;
        out[5 * i + 1] = w.n_tile;
        out[5 * i + 2] = w.kb_begin;
        out[5 * i + 3] = w.kb_end;
        out[5 * i + 4] = w.reduce ? 1u : 0u;
    }
    return (int)count;
}

extern "C" int spork_gemm_sm100_last_clock_mhz(void* stream, double* mhz)
{
    spork::DeviceState* dev = nullptr;
    const int rc = spork::current_device_state(&dev);
    if (rc) {
        return rc;
    }
    if (!mhz) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long probe[4] = {0, 0, 0, 0};
    cudaError_t e = cudaMemcpyAsync(probe, dev->status_word + 4, sizeof(probe), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(s);
    }
    if (e != cudaSuccess) {
        return (int)e;
    }
    *mhz = probe[3] > probe[1] ? double(probe[2] - probe[0]) / double(probe[3] - probe[1]) * 1e3 : 0.0;
    return 0;
}

extern "C" int spork_gemm_sm100_tune(int stages, int group_m, int l2_hints, int backoff_ns)
{
    if (stages < 0 || group_m < 0 || l2_hints < 0 || l2_hints > 0x3FFFFFF || 
        ((l2_hints >> 10) & 3) > 2 || backoff_ns < 0 || backoff_ns > 100000) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    spork::gemm_sm100::g_tuning.experiment = (l2_hints >> 4) & 15; // bits 4..7: diagnostic experiments (see Params)
    spork::gemm_sm100::g_tuning.k_atoms = (l2_hints >> 8) & 3;     // bits 8..9: column blocks per stage, 0 = choose
    spork::gemm_sm100::g_tuning.wide = (l2_hints >> 10) & 3;       // bits 10..11: 256 x 512 tiles: choose / never / always
    spork::gemm_sm100::g_tuning.wide_skew = (l2_hints >> 12) & 15; // bits 12..15: their skew, 0 = default
    spork::gemm_sm100::g_tuning.wide_group_m = (l2_hints >> 16) & 255;  // bits 16..23: their raster group, 0 = default
    spork::gemm_sm100::g_tuning.no_early_launch = (l2_hints >> 24) & 1; // bit 24: plain stream order, no early set-up
    spork::gemm_sm100::g_tuning.narrow = (l2_hints >> 25) & 1;          // bit 25: never narrow the tile to fill the machine
    l2_hints &= 15;   // bit 3 = "no hints at all" must survive (see effective_l2_hints)
    spork::gemm_sm100::g_tuning.stages = stages;
    spork::gemm_sm100::g_tuning.group_m = group_m == 0 ? spork::gemm_sm100::kGroupM : group_m;
    spork::gemm_sm100::g_tuning.l2_hints = l2_hints;
    spork::gemm_sm100::g_tuning.backoff_ns = backoff_ns;
    return 0;
}

extern "C" int spork_gemm_sm100_choice(uint32_t M, uint32_t N, uint32_t K, int variant, int split_k, int sm_count, int tf32,
                                       int* out)
{
    int block_n = variant;
    if (variant == 0) {
        block_n = N <= 64 ? 64 : (N <= 128 ? 128 : 256);
    }
    if (!out || sm_count < 2 || (block_n != 64 && block_n != 128 && block_n != 256 && block_n != 512)) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    spork::gemm_sm100::TileChoice c;
    if (!spork::gemm_sm100::choose_tile(c, M, N, K, block_n, variant == 0 ? 0 : SPORK_DEFAULT_CTA_GROUP, split_k, 0,
                                        sm_count, tf32 != 0, 1)) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    out[0] = c.block_n;
    out[1] = c.cta_group;
    out[2] = c.k_atoms;
    out[3] = c.split_k;
    return 0;
}

extern "C" int spork_gemm_sm100_tmap_cache_stats(uint64_t* hits, uint64_t* misses)
{
    if (!hits || !misses) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    *hits = spork::gemm_sm100::g_tmap_hits.load();
    *misses = spork::gemm_sm100::g_tmap_misses.load();
    return 0;
}

extern "C" int spork_gemm_sm100_stream_k_counters(uint32_t* out, void* stream)
{
    if (!out) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    spork::DeviceState* dev = nullptr;
    const int rc = spork::current_device_state(&dev);
    if (rc) {
        return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(out, dev->status_word + spork::DeviceState::kSkCounterWord0,
                                    sizeof(uint32_t) * 2 * spork::DeviceState::kSkCounters, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(s);
    }
    return (int)e;
}

extern "C" int spork_gemm_sm100_trace(void* device_buffer, uint32_t items)
{
    if ((device_buffer == nullptr) != (items == 0) || (reinterpret_cast<uintptr_t>(device_buffer) & 7u)) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    spork::gemm_sm100::g_tuning.trace = static_cast<unsigned long long*>(device_buffer);
    spork::gemm_sm100::g_tuning.trace_items = items;
    return 0;
}

extern "C" int spork_gemm_sm100_tuning(int* out, int capacity)
{
    if (!out || capacity < 10) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    const spork::gemm_sm100::Tuning t = spork::gemm_sm100::g_tuning;
    const int vals[10] = {t.stages, t.group_m, (int)spork::gemm_sm100::effective_l2_hints(t.l2_hints), t.backoff_ns,
                          t.experiment, t.k_atoms, t.wide, t.wide_skew, t.wide_group_m, t.no_early_launch};
    for (int i = 0; i < 10; ++i) {
        out[i] = vals[i];
    }
    return 0;
}

extern "C" int spork_gemm_sm100_supports(uint32_t M, uint32_t N, uint32_t K)
{
    (void)M;
    (void)N;
    return K % 8 == 0 ? 1 : 0;
}

extern "C" int spork_gemm_sm100_f16f32_ex(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C,
                                          int block_n, int cta_group, int split_k, int max_ctas, void* stream)
{
    if (cta_group < 0 || cta_group > 2 || (block_n == 0 && cta_group != 0)) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    if (block_n == 0) {
        block_n = N <= 64 ? 64 : (N <= 128 ? 128 : 256);  // the default entry point's starting width
    }
    return spork::gemm_sm100::dispatch(M, N, K, A, B, C, block_n, cta_group, split_k, max_ctas,
                                       static_cast<cudaStream_t>(stream));
}

extern "C" int spork_gemm_sm100_tf32f32(uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B, float* C,
                                        int variant, int split_k, void* stream)
{
    int block_n = variant;
    if (variant == 0) {
        block_n = N <= 64 ? 64 : (N <= 128 ? 128 : 256);
    }
    if (block_n != 64 && block_n != 128 && block_n != 256 && block_n != 512) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    return spork::gemm_sm100::dispatch(M, N, K, A, B, C, block_n, variant == 0 ? 0 : 2, split_k, 0,
                                       static_cast<cudaStream_t>(stream), true);
}

extern "C" int spork_gemm_sm100_f16f32_batched(uint32_t L, uint32_t M, uint32_t N, uint32_t K, const void* A,
                                               const void* B, float* C, int variant, int split_k, void* stream)
{
    int block_n = variant;
    if (variant == 0) {
        block_n = N <= 64 ? 64 : (N <= 128 ? 128 : 256);
    }
    if ((block_n != 64 && block_n != 128 && block_n != 256) || split_k < 0) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    return spork::gemm_sm100::dispatch(M, N, K, A, B, C, block_n, variant == 0 ? 0 : SPORK_DEFAULT_CTA_GROUP, split_k,
                                       0, static_cast<cudaStream_t>(stream), false, L);
}

extern "C" int spork_gemm_sm100_f16f32(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C,
                                       int variant, void* stream)
{
    int block_n = variant;
    if (variant == 0) {
        block_n = N <= 64 ? 64 : (N <= 128 ? 128 : 256);
    }
    if (block_n != 64 && block_n != 128 && block_n != 256 && block_n != 512) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    return spork::gemm_sm100::dispatch(M, N, K, A, B, C, block_n, variant == 0 ? 0 : SPORK_DEFAULT_CTA_GROUP, 1, 0,
                                       static_cast<cudaStream_t>(stream));
}
