// 256 x 512 output tiles per CTA pair: the large-problem variant of the sm_100a GEMM.
//
// Why: with uniform random operands the 256 x 256 kernel runs into the board's power limit, and a
// third of that power moves operand bytes from L2 into shared memory (every CTA pulls 32 KB per
// 64-deep K step).  A 256 x 512 tile needs A once for two 256-column halves of B: 48 KB per CTA for
// twice the FLOPs, a quarter fewer bytes per FLOP, and a wave of tiles touches fewer distinct strips
// of A and B, so DRAM reads fall as well.
//
// The two halves H0, H1 of a tile are two 256-column accumulators that fill all 512 columns of
// tensor memory, so there is no second buffer to hide the epilogue behind.  Instead the MMA order
// is skewed at both ends of a tile: the last G K-blocks are issued for H0 first (its accumulator is
// then final and the epilogue takes it) and only then for H1; the next tile begins with G K-blocks
// of H0 alone, into the columns just freed, while H1 is being taken.  In between, H0 and H1
// alternate per K-block so that a ring stage is released as soon as possible.  G is bounded by the
// ring depth (4 stages of 48 KB).
//
// The epilogue warps (8) copy a half accumulator from tensor memory into registers in one go
// (128 fp32 per thread) and release the columns at once: the tensor pipe waits for the copy into
// registers, not for the stores.  H0 is then written out (a swizzled shared-memory slab per warp and
// TMA stores) 32 columns at a time, and the registers each chunk frees take the same chunk of H1, so
// H1's columns are released as H0's last store is issued.  Measured on CTA 0 (spork_gemm_sm100_trace),
// 8192^3 at 1.4 GHz: copy of a half 2000-2800 cycles (128 KB per SM at the 64 bytes per clock tensor memory
// delivers into registers; one 128-column load instruction or four of 32 columns make no difference, nor
// does a sleep between the polls of the waiting issuer), write-out of a half 3500-4000 cycles; the tensor
// pipe idles about 4500 cycles per 135,000-cycle tile.
//
// Same operand layout, tensor maps, work-item list, raster and bounded waits as gemm_kernel.
#pragma once

namespace spork {
namespace gemm_sm100 {

constexpr int kWideHalfN = 256;               // columns of one accumulator half = N of one MMA
constexpr int kWideN = 2 * kWideHalfN;        // columns of a tile
constexpr int kWideEpiWarps = 8;
constexpr int kWideThreads = 32 * (2 + kWideEpiWarps);
constexpr int kWideStages = 4;
constexpr int kWideGroupM = 12;   // raster group (m-tiles); 8 / 12 / 16 measured within 1 % of each other

struct WideConfig {
    static constexpr int kABytes = kBlockM * kBlockK * 2;               // this CTA's 128 rows of A
    static constexpr int kBHalfBytes = (kWideHalfN / 2) * kBlockK * 2;  // this CTA's 128 rows of one half of B
    static constexpr int kStageBytes = kABytes + 2 * kBHalfBytes;       // 48 KB
    static constexpr int kStagingBytes = kWideEpiWarps * kSlabBytes;    // one slab per epilogue warp
    static constexpr int kBarrierBytes = 1024;
    static constexpr int kSmemBytes = 1024 + kWideStages * kStageBytes + kStagingBytes + kBarrierBytes;
    static constexpr int kTmemCols = 512;
    static_assert(kSmemBytes <= kMaxSmem, "shared memory limit");
};

struct WideBarriers {
    uint64_t full[kWideStages];
    uint64_t empty[kWideStages];
    uint64_t tmem_full[2];    // one per accumulator half
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

template <bool kTf32>
__global__ void __launch_bounds__(kWideThreads, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const Params p)
{
    using Cfg = WideConfig;
    constexpr int CG = 2;
    extern __shared__ uint8_t smem_raw[];

    const uint32_t warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x / 32, 0);
    const uint32_t lane = threadIdx.x % 32;
    const uint32_t cta_rank = cluster_ctarank();
    const bool is_leader = cta_rank == 0;
    const uint32_t group_id = blockIdx.x / CG;
    const uint32_t num_groups = gridDim.x / CG;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ring_base = smem_base;
    const uint32_t staging_base = ring_base + kWideStages * Cfg::kStageBytes;
    WideBarriers* bars =
        reinterpret_cast<WideBarriers*>(smem_raw + (staging_base + Cfg::kStagingBytes - smem_u32(smem_raw)));
    volatile uint32_t* abort_flag = &bars->abort_flag;

    unsigned long long* probe = reinterpret_cast<unsigned long long*>(p.status + 4);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kWideStages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(smem_u32(&bars->tmem_full[h]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[h]), kWideEpiWarps * CG);
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
    cluster_arrive_release();   // the peer's barriers must exist before anything arrives on them
    cluster_wait_acquire();
    tcgen05_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    const Checker chk{p.status, smem_base, smem_u32(smem_raw) + (uint32_t)Cfg::kSmemBytes, tmem_base,
                      (uint32_t)Cfg::kTmemCols};
    constexpr uint32_t kOperandBytes = kTf32 ? 4u : 2u;

    // set-up done: from here on global memory is touched, so the previous kernel in the stream must be
    // complete (see gemm_kernel)
    grid_launch_dependents();
    grid_dependency_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        probe[0] = (unsigned long long)clock64();
        probe[1] = global_timer_ns();
    }

    const uint32_t num_items = group_item_count(p, group_id, num_groups);
    constexpr int kElemsK = kTf32 ? kBlockKTf32 : kBlockK;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            const uint64_t pol_a = (p.l2_hints & 1u) ? l2_policy_evict_last() : l2_policy_evict_normal();
            const uint64_t pol_b = (p.l2_hints & 2u) ? l2_policy_evict_last()
                                   : (p.l2_hints & 4u) ? l2_policy_evict_first() : l2_policy_evict_normal();
            for (uint32_t item = 0; item < num_items && ok; ++item) {
                const WorkItem w = group_item(p, group_id, num_groups, item);
                const int32_t a_row = (int32_t)(w.m_tile * (kBlockM * CG) + cta_rank * kBlockM);
                const int32_t b_row = (int32_t)(w.n_tile * kWideN + cta_rank * (kWideHalfN / 2));
                for (uint32_t kb = w.kb_begin; kb < w.kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag, p.backoff_ns)) {
                        report_timeout(p, abort_flag, 1, stage);
                        ok = false;
                        break;
                    }
                    const uint32_t sa = ring_base + stage * Cfg::kStageBytes;
                    const uint32_t sb = sa + Cfg::kABytes;
                    const uint32_t full = smem_u32(&bars->full[stage]);
                    if (is_leader) {
                        mbar_arrive_expect_tx(full, Cfg::kStageBytes * 2);  // both CTAs' bytes land on the leader's barrier
                    }
                    const uint32_t leader_full = map_to_cta(full, 0);
                    const int32_t x = (int32_t)(kb * kElemsK);
                    if (!(chk.smem(sa, Cfg::kStageBytes, 1024u, 0x11) && chk.tma_coords(x, kOperandBytes, a_row, 0, 0x12) &&
                          chk.tma_coords(x, kOperandBytes, b_row + kWideHalfN, 0, 0x13))) {
                        *abort_flag = 1u;
                        ok = false;
                        break;
                    }
                    tma_load_2d_pair_hint(sa, &tmap_a, leader_full, x, a_row, pol_a);
                    tma_load_2d_pair_hint(sb, &tmap_b, leader_full, x, b_row, pol_b);
                    tma_load_2d_pair_hint(sb + Cfg::kBHalfBytes, &tmap_b, leader_full, x, b_row + kWideHalfN, pol_b);
                    if (++stage == kWideStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (is_leader) {
            const bool elected = elect_one();
            constexpr uint32_t idesc = kTf32 ? umma_idesc_tf32_f32(kBlockM * CG, kWideHalfN)
                                             : umma_idesc_f16_f32(kBlockM * CG, kWideHalfN);
            const uint32_t skew = p.wide_skew < 1u ? 1u : (p.wide_skew > (uint32_t)kWideStages ? (uint32_t)kWideStages
                                                                                                : p.wide_skew);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t item = 0; item < num_items && ok; ++item) {
                const WorkItem w = group_item(p, group_id, num_groups, item);
                const bool tracing = p.trace != nullptr && blockIdx.x == 0 && item < p.trace_items;
                const uint32_t n = w.kb_end - w.kb_begin;
                const uint32_t tile_phase = item & 1u;
                uint32_t done = 0;
                while (done < n && ok) {
                    const uint32_t g = wide_chunk(n, done, skew);
                    const bool first = done == 0;
                    const bool last = done + g == n;
#pragma unroll 1
                    for (uint32_t h = 0; h < 2; ++h) {
                        if (first) {
                            // the epilogue must have taken this half of the previous tile
                            // (this wait lasts thousands of cycles at every tile end while the epilogue warps
                            // work through the same memory-instruction queue: it may sleep between polls)
                            if (!__all_sync(0xFFFFFFFFu, mbar_wait<true>(smem_u32(&bars->tmem_empty[h]),
                                                                         tile_phase ^ 1u, abort_flag, p.backoff_ns))) {
                                if (elected) {
                                    report_timeout(p, abort_flag, 2, 0x40 + h);
                                }
                                ok = false;
                                break;
                            }
                            tcgen05_fence_after();
                        }
                        if (first && tracing && elected) {
                            p.trace[8 * item + h] = (unsigned long long)clock64();  // [0], [1]: this half was free
                        }
                        const uint32_t tmem_d = tmem_base + h * kWideHalfN;
                        uint32_t s = stage, ph = phase;
                        for (uint32_t j = 0; j < g; ++j) {
                            if (h == 0) {
                                if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag))) {
                                    if (elected) {
                                        report_timeout(p, abort_flag, 2, s);
                                    }
                                    ok = false;
                                    break;
                                }
                                tcgen05_fence_after();
                            }
                            const uint32_t sa = ring_base + s * Cfg::kStageBytes;
                            if (!(chk.smem(sa, Cfg::kStageBytes, 1024u, 0x21) && chk.tmem(tmem_d, kWideHalfN, 0x22))) {
                                *abort_flag = 1u;
                                ok = false;
                                break;
                            }
                            if (elected) {
                                const uint64_t desc_a = umma_desc_kmajor_sw128(sa);
                                const uint64_t desc_b = umma_desc_kmajor_sw128(sa + Cfg::kABytes + h * Cfg::kBHalfBytes);
#pragma unroll
                                for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                                    const uint32_t acc = (!first || j != 0 || k != 0) ? 1u : 0u;
                                    if (kTf32) {
                                        umma_tf32_ss<CG>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc, acc);
                                    } else {
                                        umma_f16_ss<CG>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc, acc);
                                    }
                                }
                                if (h == 1) {
                                    // both halves have read the stage: free it in both CTAs
                                    const uint32_t empty = smem_u32(&bars->empty[s]);
                                    umma_commit<CG>(empty);
                                    umma_commit<CG>(map_to_cta(empty, 1));
                                }
                            }
                            if (++s == kWideStages) {
                                s = 0;
                                ph ^= 1u;
                            }
                        }
                        if (!ok) {
                            break;
                        }
                        if (last && elected) {
                            // this half is final: wake the epilogue warps of both CTAs
                            const uint32_t tfull = smem_u32(&bars->tmem_full[h]);
                            umma_commit<CG>(tfull);
                            umma_commit<CG>(map_to_cta(tfull, 1));
                        }
                        if (h == 1) {
                            stage = s;
                            phase = ph;
                        }
                    }
                    done += g;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t quarter = warp % 4;                       // TMEM lanes [32*quarter, +32) belong to this warp
        const uint32_t part = (warp - kEpilogueWarp0) / 4;       // which 128 of a half's 256 columns
        const uint32_t slab = staging_base + (warp - kEpilogueWarp0) * kSlabBytes;
        bool ok = chk.smem(slab, kSlabBytes, 1024u, 0x32);
        uint32_t r[4][32];   // 128 accumulator columns of this thread's row
        for (uint32_t item = 0; item < num_items && ok; ++item) {
            const WorkItem w = group_item(p, group_id, num_groups, item);
            const uint32_t tile_phase = item & 1u;
            const uint32_t row0 = w.m_tile * (kBlockM * CG) + cta_rank * kBlockM + quarter * 32;
            const bool rows_live = row0 < p.M && w.kb_begin < w.kb_end;
            const bool tracing = p.trace != nullptr && blockIdx.x == 0 && warp == kEpilogueWarp0 && lane == 0 &&
                                 item < p.trace_items;
            const uint32_t taddr0 = tmem_base + ((quarter * 32u) << 16) + part * 128u;  // + h * 256 + c * 32
            const uint32_t col_base = w.n_tile * kWideN + part * 128u;                    // + h * 256 + c * 32

            // half `h` is final: a stamp, and the acquire side of the hand-over
            auto wait_full = [&](uint32_t h) {
                if (!mbar_wait(smem_u32(&bars->tmem_full[h]), tile_phase, abort_flag, p.backoff_ns)) {
                    if (lane == 0) {
                        report_timeout(p, abort_flag, 3, 0x40 + h);
                    }
                    return false;
                }
                tcgen05_fence_after();
                if (tracing) {
                    p.trace[8 * item + 2 + 3 * h] = (unsigned long long)clock64();  // [2], [5]: the half was final
                }
                return chk.tmem(taddr0 + h * kWideHalfN, 4 * kEpiCols, 0x31);
            };
            // every column of half `h` sits in registers: the issuer may overwrite it
            auto release = [&](uint32_t h) {
                tmem_ld_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(map_to_cta(smem_u32(&bars->tmem_empty[h]), 0));
                }
                if (tracing) {
                    p.trace[8 * item + 3 + 3 * h] = (unsigned long long)clock64();  // [3], [6]: it sits in registers
                }
            };
            // chunk c (32 columns) of half h: registers -> slab -> TMA store (or reduce-add, or guarded scalar stores)
            auto store_chunk = [&](uint32_t h, int c) {
                const uint32_t col = col_base + h * kWideHalfN + c * kEpiCols;
                if (!rows_live || col >= p.N || (p.experiment & 1u)) {
                    return;  // warp-uniform
                }
                if (p.use_tma_store && !w.reduce && (p.experiment & 8u)) {
                    // Diagnostic alternative to the TMA stores below (same results): plain stores, made
                    // whole 128-byte lines by a turn through the slab.  Eight lanes write one row of the
                    // slab (128 bytes), four rows per instruction.  Measured slower than the TMA stores
                    // on every shape, at the power limit and off it.
                    __syncwarp();
                    const uint32_t row_addr = slab + lane * 128u;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        st_shared_v4(row_addr + (((uint32_t)j ^ (lane & 7u)) << 4), r[c][4 * j], r[c][4 * j + 1],
                                     r[c][4 * j + 2], r[c][4 * j + 3]);
                    }
                    __syncwarp();
                    const uint32_t sub_row = lane >> 3, piece = lane & 7u;
                    const uint32_t gcol = col + piece * 4u;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t srow = 4u * i + sub_row;
                        const uint4 v = ld_shared_v4(slab + srow * 128u + ((piece ^ (srow & 7u)) << 4));
                        const uint32_t grow = row0 + srow;
                        if (grow < p.M && gcol < p.N) {
                            st_global_v4(p.C + (size_t)grow * p.N + gcol, v);
                        }
                    }
                } else if (p.use_tma_store) {
                    if (lane == 0) {
                        bulk_wait_group_read<0>();  // the previous store has read the slab
                    }
                    __syncwarp();
                    const uint32_t row_addr = slab + lane * 128u;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        st_shared_v4(row_addr + (((uint32_t)j ^ (lane & 7u)) << 4), r[c][4 * j], r[c][4 * j + 1],
                                     r[c][4 * j + 2], r[c][4 * j + 3]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (w.reduce) {
                            tma_reduce_add_2d(&tmap_c, slab, (int32_t)col, (int32_t)row0);
                        } else {
                            tma_store_2d(&tmap_c, slab, (int32_t)col, (int32_t)row0);
                        }
                        bulk_commit_group();
                    }
                } else {
                    const uint32_t row = row0 + lane;
                    if (row < p.M) {
                        float* dst = p.C + (size_t)row * p.N + col;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (col + j < p.N) {
                                if (w.reduce) {
                                    atomicAdd(dst + j, __uint_as_float(r[c][j]));
                                } else {
                                    dst[j] = __uint_as_float(r[c][j]);
                                }
                            }
                        }
                    }
                }
            };

            // H0: tensor memory -> registers, release
            if (!wait_full(0)) {
                ok = false;
                break;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                tmem_ld_32x32b_x32(taddr0 + c * kEpiCols, r[c]);
            }
            release(0);
            // H1 became final while that copy ran (it trails H0 by the skew).  Write H0 out chunk by chunk and
            // refill each chunk's registers with H1 at once, so that H1's columns are free when H0's last store
            // has been issued, not a second copy later.
            if (!wait_full(1)) {
                ok = false;
                break;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                store_chunk(0, c);
                tmem_ld_32x32b_x32(taddr0 + kWideHalfN + c * kEpiCols, r[c]);
            }
            if (tracing) {
                p.trace[8 * item + 4] = (unsigned long long)clock64();  // [4]: H0's last store was issued
            }
            release(1);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                store_chunk(1, c);
            }
            if (tracing) {
                p.trace[8 * item + 7] = (unsigned long long)clock64();  // [7]: H1's last store was issued
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
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<CG>(tmem_base, Cfg::kTmemCols);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        probe[2] = (unsigned long long)clock64();
        probe[3] = global_timer_ns();
    }
}

}  // namespace gemm_sm100
}  // namespace spork
