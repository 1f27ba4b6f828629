// Attention forward for sm_100a (B200): O = softmax(Q K^T * scale) V per head,
// fp16 or bfloat16 in and out, fp32 softmax, optionally with a causal mask.
//
// Takes the place of the reference's attention launch entry
// (launch_tk_4090_fwd_kernel / htod_f32_tk_4090_fwd, tk_4090_fwd.hpp:5-7; the
// kernel source itself is not part of the reference tree) and computes the
// math of simple_attn (torch_attn.py:11-16).
//
// One CTA owns TWO 128-row query tiles of one head and streams the head's keys
// and values through them in blocks of 128, FlashAttention style:
//   warps 0-3  softmax of query tile 0 (one thread = one query row)
//   warps 4-7  softmax of query tile 1
//   warp  8    TMA producer (Q tiles once, then K_j, V_j through a ring)
//   warp  9    tcgen05.mma issuer (the whole warp runs the control flow, an elected lane issues) and TMEM owner
//   warps 10-11 idle: they complete the third warpgroup, so that whole warpgroups can trade
//              registers (setmaxnreg): 216 per softmax thread, 72 for the rest
// Tensor memory (512 columns): score buffers of 128 fp32 columns, then O0 | O1 of D columns each.  Head
// dimension 128: two score buffers, one per query tile.  Head dimension 64: three, used in rotation by the
// (tile, block) pairs in issue order, so the next score tile of a query tile is ready before its softmax
// has finished the current one (see Config::kScoreBufs).
// Per key block j and query tile w:
//   S_w = Q_w K_j^T            tcgen05.mma, both operands K-major in shared memory
//   softmax thread: reads its whole S row into registers, row max,
//       p = exp2((s - m) * scale*log2e) (five of every eight pairs by ex2.approx, three by a
//       cubic on the multiply-add pipe: the special-function unit is the softmax's bound),
//       row sum; P_w (fp16, two per column) is
//       written back into tensor memory over the first 64 columns of S_w and handed to the
//       issuer in two halves of 64 keys, so the first half is multiplied while the second is
//       still being exponentiated;
//       O_w is rescaled in place (tcgen05.ld/st), before the first half is handed over, only
//       when the row max grew by more than 2^8 since the last rescale (p then stays within
//       fp16 range)
//   O_w += P_w V_j             tcgen05.mma, A = P_w from tensor memory, B = V_j (N-major)
// The two query tiles alternate, so the tensor core works on one tile while the
// other tile's softmax runs.  With a causal mask each tile stops at its own diagonal block.
// Keys past the end of a ragged sequence are masked
// to -inf; rows past the end are computed on zero-filled queries and not stored.
// Every wait on a barrier is bounded (see ptx_sm100.cuh); the one wait that is not, setmaxnreg's for free
// registers, cannot block because the trade fits the launch allocation (static_assert below).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <math.h>
#include <mutex>
#include <stdint.h>
#include <stdio.h>

#include "../../include/spork_b200.h"
#include "device_state.h"
#include "ptx_sm100.cuh"

namespace spork {
namespace attn_sm100 {

using namespace ptx;

constexpr int kTileQ = 128;     // query rows per tile (= TMEM lanes)
constexpr int kTileKV = 128;    // keys per block
constexpr int kNumThreads = 384;     // 8 softmax warps, the TMA warp, the MMA warp, two idle warps that complete the third warpgroup
constexpr int kSoftmaxRegs = 216;    // registers per thread after the warpgroups trade: 2*128*232 + 128*40 <= 64 Ki
constexpr int kOtherRegs = 72;
// setmaxnreg.inc waits, without a limit, for registers to be free: the trade must fit the allocation the
// CTA was launched with (kNumThreads * 168), not the whole file
static_assert(2 * kSoftmaxRegs + kOtherRegs <= 3 * 168, "register trade exceeds the launch allocation");
constexpr int kLoadWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kMaxKvStages = 8;
constexpr int kTmemCols = 512;
constexpr uint32_t kSoftmaxBackoffNs = 20;  // the softmax warps' waits sleep between polls
constexpr float kRescaleThreshold = 8.0f;  // log2 units: rescale O only when the max grew by more than 2^8

template <int D>
struct Config {
    static_assert(D == 64 || D == 128, "head dimension");
    static constexpr int kAtoms = D / 64;                      // 64-wide (128-byte) column blocks of a tile
    static constexpr int kTileBytes = kTileQ * D * 2;          // a Q, K or V tile
    static constexpr int kAtomBytes = 128 * 128;               // 128 rows x 128 bytes
    static constexpr int kStagesFit = (227 * 1024 - 2048 - 2 * kTileBytes) / kTileBytes;
    static constexpr int kKvStages = kStagesFit > kMaxKvStages ? kMaxKvStages : kStagesFit;
    static constexpr int kSmemBytes = 1024 + 2 * kTileBytes + kKvStages * kTileBytes + 1024;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory limit");
    // Score buffers in tensor memory, 128 fp32 columns each, used in rotation by the (query tile, key block)
    // pairs in issue order.  With head dimension 128 the two O accumulators take half of tensor memory and two
    // buffers remain: one per query tile, and S_w(j+1) can only be issued once P_w(j) V_j has consumed the
    // buffer.  With head dimension 64 the accumulators take 128 columns and a third buffer fits: the next
    // score tile is computed while the previous one is still being exponentiated, so a query tile's softmax
    // goes from block to block without waiting for the tensor core.
    static constexpr int kScoreBufs = D == 64 ? 3 : 2;
    static_assert(kScoreBufs * 128 + 2 * D <= kTmemCols, "tensor memory budget");
};

struct Params {
    int BH, S, D;
    int q_pairs;        // ceil(S / 256): CTAs per head
    int kv_blocks;      // ceil(S / 128)
    int causal;         // 1: key j contributes to query i only if j <= i
    float scale_log2e;  // scale * log2(e)
    void* o;            // fp16 or bf16, [BH][S][D]
    uint32_t* status;
};

struct Barriers {
    uint64_t q_full;
    uint64_t kv_full[kMaxKvStages];
    uint64_t kv_empty[kMaxKvStages];
    uint64_t s_full[3];      // per score buffer
    uint64_t p_ready[3][2];  // [score buffer][key half]
    uint64_t pv_done[2];     // per query tile
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// the two-buffer kernel's barriers
struct BarriersTwo {
    uint64_t q_full;
    uint64_t kv_full[kMaxKvStages];
    uint64_t kv_empty[kMaxKvStages];
    uint64_t s_full[2];
    uint64_t p_ready[2][2];  // [query tile][key half]
    uint64_t pv_done[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Largest of three: one instruction of the 16-lane integer/logic pipe where two-input max needs two.
__device__ __forceinline__ float max3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ float fma_sat(float a, float b, float c)
{
    float r;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// 2^x for a pair of scores on the fused-multiply-add pipe instead of the special-function unit, which
// at 8 cycles per warp instruction is what bounds the softmax. x = s*sl2 + neg_m is formed clamped to
// [-kPolyLo, 8] by a saturating multiply-add (y = (x + kPolyLo) / 64 in [0, 1]; the upper end is never
// reached because the lazy rescaling keeps x <= 8), split into round(x) and a fraction in [-1/2, 1/2] by
// the 1.5*2^23 trick, the fraction goes through a cubic (relative error 7e-5, well under the rounding of P
// to 16 bits) and round(x) is added into the exponent field. ks = sl2 / 64, cs = (neg_m + kPolyLo) / 64.
constexpr float kPolyLo = 56.0f;
// How many of every eight pairs of exponentials take that route. Measured at B*H = 256, S = 4096, D = 128,
// interleaved runs on a part warmed into its power cap: 0 -> 1099, 1 -> 1145, 2 -> 1163, 3 -> 1173,
// 4 -> 1069 TFLOP/s (cold: 1264, 1281, 1173, 1193, 1112).
#ifndef SPORK_ATTN_POLY_PAIRS_D128
#define SPORK_ATTN_POLY_PAIRS_D128 3
#endif
#ifndef SPORK_ATTN_POLY_PAIRS_D64
#define SPORK_ATTN_POLY_PAIRS_D64 3
#endif
template <int D>
constexpr int kPolyPairs = D == 64 ? SPORK_ATTN_POLY_PAIRS_D64 : SPORK_ATTN_POLY_PAIRS_D128;
__device__ __forceinline__ void ex2_poly2(float s0, float s1, float ks, float cs, float& p0, float& p1)
{
    const uint64_t y = pack2(fma_sat(s0, ks, cs), fma_sat(s1, ks, cs));
    const uint64_t c64 = pack2(64.0f, 64.0f);
    const uint64_t magic = pack2(12582912.0f - kPolyLo, 12582912.0f - kPolyLo);
    const uint64_t t = fma2(y, c64, magic);                       // 1.5*2^23 + round(x)
    const uint64_t nr = fma2(t, pack2(-1.0f, -1.0f), magic);      // -(round(x) + kPolyLo)
    const uint64_t f = fma2(y, c64, nr);                          // x - round(x)
    uint64_t q = fma2(f, pack2(0.0551716648f, 0.0551716648f), pack2(0.2426111251f, 0.2426111251f));
    q = fma2(q, f, pack2(0.6932609677f, 0.6932609677f));
    q = fma2(q, f, pack2(0.9999280572f, 0.9999280572f));
    float t0, t1, q0, q1;
    unpack2(t, t0, t1);
    unpack2(q, q0, q1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

// Two fp32 values rounded to a packed pair of 16-bit floats (low half first): fp16 or bf16.
template <bool kBf16>
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
{
    if (kBf16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void report_timeout(const Params& p, volatile uint32_t* abort_flag, uint32_t role,
                                               uint32_t where)
{
    *abort_flag = 1u;
    atomicCAS(p.status, 0u, 0x90000000u | (role << 24) | ((where & 0xFFu) << 16) | (blockIdx.x & 0xFFFFu));
}

// ---------------------------------------------------------------------------------------------------
// The two-buffer kernel (head dimension 128): score buffer w belongs to query tile w, S_w(j+1) is issued
// after P_w(j) V_j has consumed the buffer.  kCausal: compiled with the mask, each tile stopping at its own
// diagonal block (the non-causal instance carries none of that code).  It is kept as a kernel of its own, apart from the
// rotating-buffer kernel below that head dimension 64 uses: with everything about a tile a compile-time
// offset its MMA issuer is a few instructions per multiply, and measured on the same box it is 4-7 %
// faster at head dimension 128 than the general kernel run with two buffers (the kernel is sensitive to
// the issuer's instruction count and to instruction-cache pressure on the issuer's sub-partition).
// kBf16: Q, K, V, P and O are bfloat16 (the reference interface's type, matrix_util.hpp:40-45) instead of fp16.
template <int D, bool kBf16, bool kCausal>
__global__ void __launch_bounds__(kNumThreads, 1)
attn_fwd_two_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const Params p)
{
    using Cfg = Config<D>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x / 32, 0);  // provably the same in all lanes
    const uint32_t lane = threadIdx.x % 32;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;                                  // 2 Q tiles
    const uint32_t kv_smem = q_smem + 2 * Cfg::kTileBytes;              // ring of K / V tiles
    constexpr int kKvStages = Cfg::kKvStages;
    BarriersTwo* bars =
        reinterpret_cast<BarriersTwo*>(smem_raw + (kv_smem + kKvStages * Cfg::kTileBytes - smem_u32(smem_raw)));
    volatile uint32_t* abort_flag = &bars->abort_flag;

    // Clock probe: the last CTA notes SM cycles and wall-clock nanoseconds at both ends of its life; their
    // ratio is the SM clock this launch really ran at late in its run (read by spork_gemm_sm100_last_clock_mhz).
    unsigned long long* probe = reinterpret_cast<unsigned long long*>(p.status + 4);
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
        probe[0] = (unsigned long long)clock64();
        probe[1] = global_timer_ns();
    }

    const int head = blockIdx.x / p.q_pairs;
    // causal: the pairs with the most key blocks are launched first, so the short ones fill the tail
    const int q_pair = kCausal ? p.q_pairs - 1 - (int)(blockIdx.x % p.q_pairs) : (int)(blockIdx.x % p.q_pairs);
    const int q_row0 = q_pair * 2 * kTileQ;
    // causal: keys beyond a tile's last query row are never needed, so the first tile stops one block
    // before the second (n_blocks0 = n_blocks - 1, or the same when the second tile lies past the end)
    const int last_row = q_row0 + 2 * kTileQ - 1 < p.S - 1 ? q_row0 + 2 * kTileQ - 1 : p.S - 1;
    const int last_row0 = q_row0 + kTileQ - 1 < p.S - 1 ? q_row0 + kTileQ - 1 : p.S - 1;
    const int n_blocks = kCausal ? last_row / kTileKV + 1 : p.kv_blocks;
    const int n_blocks0 = kCausal ? last_row0 / kTileKV + 1 : n_blocks;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->q_full), 1);
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(smem_u32(&bars->kv_full[s]), 1);
            mbar_init(smem_u32(&bars->kv_empty[s]), 1);
        }
        for (int w = 0; w < 2; ++w) {
            mbar_init(smem_u32(&bars->s_full[w]), 1);
            for (int h = 0; h < 2; ++h) {
                mbar_init(smem_u32(&bars->p_ready[w][h]), kTileQ);
            }
            mbar_init(smem_u32(&bars->pv_done[w]), 1);
        }
        bars->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == kLoadWarp && lane == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
    }
    if (warp == kMmaWarp) {
        tmem_alloc<1>(smem_u32(&bars->tmem_base), kTmemCols);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    // column offsets inside the allocation
    const uint32_t tmem_s0 = tmem_base;          // S_w at + w * 128; P_w (fp16 pairs) reuses its first 64 columns
    const uint32_t tmem_o0 = tmem_base + 256;    // O_w at + w * 128

    // The softmax keeps a whole row of 128 scores in registers and needs room beside them to overlap
    // the exponentials' latencies; the loader and the issuer need almost none. Whole warpgroups trade.
    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
        if (warp == kLoadWarp) {
        // ---------------------------------------------------------- TMA producer
        if (lane == 0) {
            const uint32_t qf = smem_u32(&bars->q_full);
            mbar_arrive_expect_tx(qf, 2 * Cfg::kTileBytes);
            for (int w = 0; w < 2; ++w) {
                for (int a = 0; a < Cfg::kAtoms; ++a) {
                    tma_load_3d(q_smem + w * Cfg::kTileBytes + a * Cfg::kAtomBytes, &tmap_q, qf, a * 64,
                                q_row0 + w * kTileQ, head);
                }
            }
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = 0; t < 2 * n_blocks && ok; ++t) {
                // tile order: K_0, V_0, K_1, V_1, ...
                const int j = t >> 1;
                const CUtensorMap* map = (t & 1) ? &tmap_v : &tmap_k;
                if (!mbar_wait(smem_u32(&bars->kv_empty[stage]), phase ^ 1u, abort_flag)) {
                    report_timeout(p, abort_flag, 1, stage);
                    ok = false;
                    break;
                }
                const uint32_t full = smem_u32(&bars->kv_full[stage]);
                mbar_arrive_expect_tx(full, Cfg::kTileBytes);
                for (int a = 0; a < Cfg::kAtoms; ++a) {
                    tma_load_3d(kv_smem + stage * Cfg::kTileBytes + a * Cfg::kAtomBytes, map, full, a * 64,
                                j * kTileKV, head);
                }
                if (++stage == (uint32_t)kKvStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the control flow and one elected lane issues. Everything an issue needs
        // (descriptors, tensor-memory and barrier addresses) is then the same in all lanes and can live in
        // uniform registers; issued from inside a one-lane branch each multiply cost the thread about
        // 60 cycles, as long as the tensor core needs to execute it, and the issuer bounded the kernel.
        const bool leader = elect_one();
        constexpr uint32_t idesc_qk = umma_idesc_f16_f32(kTileQ, kTileKV, false, false, kBf16);
        constexpr uint32_t idesc_pv = umma_idesc_f16_f32(kTileQ, D, false, true, kBf16);  // B = V is N-major
        uint32_t stage = 0, phase = 0;  // ring position of the next tile to consume
        bool ok = true;
        auto advance = [&]() {
            if (++stage == (uint32_t)kKvStages) {
                stage = 0;
                phase ^= 1u;
            }
        };
        // Descriptor low words: one per operand tile, advanced by compile-time constants per MMA
        // (a 64-wide column block further = +1024, 16 elements along K inside a block = +2,
        // 16 rows further down an N-major V tile = +128, all in units of 16 bytes).
        const uint32_t q_lo0 = desc_lo_kmajor(q_smem);
        // S_w = Q_w K^T from the K tile in ring slot `st`. (Not split along the keys: with both operands
        // in shared memory a 128 x 64 x 16 step reads 6 KB in 32 cycles, more than shared memory delivers.)
        auto issue_qk = [&](int w, uint32_t st) {
            const uint32_t k_lo = desc_lo_kmajor(kv_smem + st * Cfg::kTileBytes);
            const uint32_t q_lo = q_lo0 + (uint32_t)w * (Cfg::kTileBytes >> 4);
            if (leader) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (uint32_t)((kk / 4) * (Cfg::kAtomBytes >> 4) + 2 * (kk % 4));
                    umma_f16_ss_cta1(tmem_s0 + w * 128, q_lo + off, kDescHiSw128, k_lo + off, kDescHiSw128, idesc_qk,
                                     kk != 0 ? 1u : 0u);
                }
                umma_commit<1>(smem_u32(&bars->s_full[w]));
            }
        };
        // O_w (+)= P_w V: A = P_w in tensor memory (16 keys = 8 packed columns per step),
        // B = the V tile in ring slot `st` (N-major; its d-halves are one 128-row block apart);
        // half h covers keys [64 h, 64 h + 64)
        auto issue_pv = [&](int w, uint32_t st, bool accumulate, int h) {
            const uint32_t v_lo = desc_lo_mnmajor(kv_smem + st * Cfg::kTileBytes, Cfg::kAtomBytes);
            if (leader) {
#pragma unroll
                for (int kk = h * (kTileKV / 32); kk < (h + 1) * (kTileKV / 32); ++kk) {
                    umma_f16_ts_cta1(tmem_o0 + w * 128, tmem_s0 + w * 128 + kk * 8, v_lo + (uint32_t)(kk * 128),
                                     kDescHiSw128, idesc_pv, (accumulate || kk != 0) ? 1u : 0u);
                }
            }
        };
        auto commit = [&](uint64_t* bar) {
            if (leader) {
                umma_commit<1>(smem_u32(bar));
            }
        };
        // every lane polls; a timeout is reported once
        auto wait = [&](uint64_t* bar, uint32_t parity, uint32_t where) {
            const bool done = mbar_wait(smem_u32(bar), parity, abort_flag);
            if (!done && leader) {
                report_timeout(p, abort_flag, 2, where);
            }
            return __all_sync(0xFFFFFFFFu, done);
        };
        do {
            if (!wait(&bars->q_full, 0, 0x20)) {
                break;
            }
            // prologue: S_0(0), S_1(0)
            if (!wait(&bars->kv_full[stage], phase, stage)) {
                break;
            }
            tcgen05_fence_after();
            issue_qk(0, stage);
            issue_qk(1, stage);
            commit(&bars->kv_empty[stage]);
            advance();
            for (int j = 0; j < n_blocks && ok; ++j) {
                const uint32_t v_stage = stage, v_phase = phase;
                advance();
                const uint32_t k_stage = stage, k_phase = phase;  // K_{j+1}, if any
                const bool more = j + 1 < n_blocks;
                if (more) {
                    advance();
                }
                // The tiles this block's multiplies read were requested long ago; make sure of them now, while
                // the softmax is still at work, so that nothing stands between P arriving and the issue.
                if (!wait(&bars->kv_full[v_stage], v_phase, v_stage) ||
                    (more && !wait(&bars->kv_full[k_stage], k_phase, k_stage))) {
                    ok = false;
                    break;
                }
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    if (!ok) {
                        break;
                    }
                    if (kCausal && w == 0 && j >= n_blocks0) {
                        continue;  // the first tile is past its diagonal
                    }
                    const bool more_w = (kCausal && w == 0) ? j + 1 < n_blocks0 : more;
                    if (!wait(&bars->p_ready[w][0], (uint32_t)(j & 1), 0x30 + w)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    issue_pv(w, v_stage, j > 0, 0);  // the first 64 keys, while the softmax does the rest
                    if (!wait(&bars->p_ready[w][1], (uint32_t)(j & 1), 0x38 + w)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    issue_pv(w, v_stage, true, 1);
                    if (more_w) {
                        issue_qk(w, k_stage);
                    } else {
                        commit(&bars->pv_done[w]);  // completes once: O_w is final
                    }
                    if (w == 1) {
                        commit(&bars->kv_empty[v_stage]);
                        if (more) {
                            commit(&bars->kv_empty[k_stage]);
                        }
                    }
                }
            }
        } while (false);
        }
    } else {
        // --------------------------------------------------------------- softmax
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
        const uint32_t w = warp / 4;        // query tile of this warpgroup
        const uint32_t quarter = warp % 4;  // TMEM lanes [32*quarter, +32)
        const uint32_t row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32u) << 16;
        const uint32_t tmem_s = tmem_s0 + w * 128 + lane_addr;
        const uint32_t tmem_o = tmem_o0 + w * 128 + lane_addr;
        const float sl2 = p.scale_log2e;
        float m_ref = -INFINITY;  // row max the stored O and l are relative to (raw scores)
        float l_run = 0.0f;       // running row sum
        bool ok = true;
        const int n_blocks_w = w == 0 ? n_blocks0 : n_blocks;
        for (int j = 0; j < n_blocks_w; ++j) {
            if (!mbar_wait(smem_u32(&bars->s_full[w]), (uint32_t)(j & 1), abort_flag, kSoftmaxBackoffNs)) {
                if (lane == 0) {
                    report_timeout(p, abort_flag, 3, 0x10 + w);
                }
                ok = false;
                break;
            }
            // A completed s_full also means every earlier MMA of the issuing thread is complete: P_w of the
            // previous block has been consumed and O_w is not being written.
            tcgen05_fence_after();
            uint32_t r[128];
            {
                uint32_t(&r0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[0]);
                uint32_t(&r1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[32]);
                uint32_t(&r2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[64]);
                uint32_t(&r3)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[96]);
                tmem_ld_32x32b_x32(tmem_s, r0);
                tmem_ld_32x32b_x32(tmem_s + 32, r1);
                tmem_ld_32x32b_x32(tmem_s + 64, r2);
                tmem_ld_32x32b_x32(tmem_s + 96, r3);
                tmem_ld_wait();
            }
            int valid = p.S - j * kTileKV;  // keys of this block that exist
            bool masked = valid < kTileKV;  // uniform over the CTA
            if (kCausal) {
                // keys of this block this row may see: global key index <= global query index
                const int row_global = q_row0 + (int)w * kTileQ + (int)row;
                const int seen = row_global - j * kTileKV + 1;
                valid = seen < valid ? seen : valid;
                masked = masked || (j + 1) * kTileKV > q_row0 + (int)w * kTileQ + 1;  // uniform over the tile
            }
            if (masked) {
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    if (i >= valid) {
                        r[i] = 0xFF800000u;  // -inf
                    }
                }
            }
            // four independent chains of three-input max
            float m4[4] = {__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]),
                           __uint_as_float(r[3])};
#pragma unroll
            for (int i = 4; i < 124; i += 8) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    m4[c] = max3(m4[c], __uint_as_float(r[i + 2 * c]), __uint_as_float(r[i + 2 * c + 1]));
                }
            }
            m4[0] = max3(m4[0], __uint_as_float(r[124]), __uint_as_float(r[125]));
            m4[1] = max3(m4[1], __uint_as_float(r[126]), __uint_as_float(r[127]));
            const float m_blk = fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]);
            // Lazy rescale: keep the old reference max unless the new one is more than 2^8 above it.
            const bool grow = j == 0 || (m_blk - m_ref) * sl2 > kRescaleThreshold;
            float alpha = 1.0f;
            if (grow) {
                alpha = ex2_approx((m_ref - m_blk) * sl2);  // 0 on the first block
                m_ref = m_blk;
            }
            // Rescale O_w when some row of this warp moved its reference max (never on the first block).
            // It has to be finished before the first half of P is handed over: from then on the issuer
            // accumulates into O_w.
            if (j > 0 && __any_sync(0xFFFFFFFFu, grow)) {
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32b_x32(tmem_o + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    }
                    tmem_st_32x32b_x32(tmem_o + c * 32, o);
                }
            }
            const float neg_m = -m_ref * sl2;
            const float ks = sl2 * (1.0f / 64.0f);
            const float cs = (neg_m + kPolyLo) * (1.0f / 64.0f);
            // packed forms where both elements of a pair take the same step: half the issue slots
            const uint64_t sl2_2 = pack2(sl2, sl2);
            const uint64_t neg_m2 = pack2(neg_m, neg_m);
            uint64_t l_blk2 = pack2(0.0f, 0.0f);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t packed[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float s0 = __uint_as_float(r[half * 64 + 2 * i]);
                    const float s1 = __uint_as_float(r[half * 64 + 2 * i + 1]);
                    float p0, p1;
                    if ((i & 7) < kPolyPairs<D>) {
                        ex2_poly2(s0, s1, ks, cs, p0, p1);
                    } else {
                        float x0, x1;
                        unpack2(fma2(pack2(s0, s1), sl2_2, neg_m2), x0, x1);
                        p0 = ex2_approx(x0);
                        p1 = ex2_approx(x1);
                    }
                    l_blk2 = add2(l_blk2, pack2(p0, p1));
                    packed[i] = pack_half2<kBf16>(p0, p1);
                }
                tmem_st_32x32b_x32(tmem_s + half * 32, packed);
                // hand this half of P_w over: the issuer multiplies it while the other half is computed
                tmem_st_wait();
                tcgen05_fence_before();
                mbar_arrive(smem_u32(&bars->p_ready[w][half]));
            }
            float l_blk0, l_blk1;
            unpack2(l_blk2, l_blk0, l_blk1);
            l_run = l_run * alpha + (l_blk0 + l_blk1);
        }
        // ---- epilogue: O_w / l -> fp16 -> global
        if (ok) {
            if (!mbar_wait(smem_u32(&bars->pv_done[w]), 0u, abort_flag, 20)) {
                if (lane == 0) {
                    report_timeout(p, abort_flag, 3, 0x28 + w);
                }
                ok = false;
            }
        }
        if (ok) {
            tcgen05_fence_after();
            const float inv_l = 1.0f / l_run;
            const int q_row = q_row0 + (int)w * kTileQ + (int)row;
            uint16_t* dst = static_cast<uint16_t*>(p.o) + ((size_t)head * p.S + (size_t)(q_row < p.S ? q_row : 0)) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_o + c * 32, r);
                tmem_ld_wait();
                if (q_row < p.S) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 v;
                        v.x = pack_half2<kBf16>(__uint_as_float(r[8 * q4 + 0]) * inv_l, __uint_as_float(r[8 * q4 + 1]) * inv_l);
                        v.y = pack_half2<kBf16>(__uint_as_float(r[8 * q4 + 2]) * inv_l, __uint_as_float(r[8 * q4 + 3]) * inv_l);
                        v.z = pack_half2<kBf16>(__uint_as_float(r[8 * q4 + 4]) * inv_l, __uint_as_float(r[8 * q4 + 5]) * inv_l);
                        v.w = pack_half2<kBf16>(__uint_as_float(r[8 * q4 + 6]) * inv_l, __uint_as_float(r[8 * q4 + 7]) * inv_l);
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = v;
                    }
                }
            }
        }
    }

    // ----------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
        probe[2] = (unsigned long long)clock64();
        probe[3] = global_timer_ns();
    }
}

// ---------------------------------------------------------------------------------------------------
// The rotating-buffer kernel (head dimension 64; it also runs with two buffers at head dimension 128).
// kBf16: Q, K, V, P and O are bfloat16 (the reference interface's type, matrix_util.hpp:40-45) instead of fp16.
template <int D, bool kBf16>
__global__ void __launch_bounds__(kNumThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const Params p)
{
    using Cfg = Config<D>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x / 32, 0);  // provably the same in all lanes
    const uint32_t lane = threadIdx.x % 32;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;                                  // 2 Q tiles
    const uint32_t kv_smem = q_smem + 2 * Cfg::kTileBytes;              // ring of K / V tiles
    constexpr int kKvStages = Cfg::kKvStages;
    Barriers* bars =
        reinterpret_cast<Barriers*>(smem_raw + (kv_smem + kKvStages * Cfg::kTileBytes - smem_u32(smem_raw)));
    volatile uint32_t* abort_flag = &bars->abort_flag;

    // Clock probe: the last CTA notes SM cycles and wall-clock nanoseconds at both ends of its life; their
    // ratio is the SM clock this launch really ran at late in its run (read by spork_gemm_sm100_last_clock_mhz).
    unsigned long long* probe = reinterpret_cast<unsigned long long*>(p.status + 4);
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
        probe[0] = (unsigned long long)clock64();
        probe[1] = global_timer_ns();
    }

    const int head = blockIdx.x / p.q_pairs;
    // causal: the pairs with the most key blocks are launched first, so the short ones fill the tail
    const int q_pair = p.causal ? p.q_pairs - 1 - (int)(blockIdx.x % p.q_pairs) : (int)(blockIdx.x % p.q_pairs);
    const int q_row0 = q_pair * 2 * kTileQ;
    // Key blocks each query tile walks.  Causal: keys beyond a tile's last query row are never needed, so
    // the first tile stops one block before the second (it used to walk a fully masked block).
    const int last_row0 = q_row0 + kTileQ - 1 < p.S - 1 ? q_row0 + kTileQ - 1 : p.S - 1;
    const int last_row1 = q_row0 + 2 * kTileQ - 1 < p.S - 1 ? q_row0 + 2 * kTileQ - 1 : p.S - 1;
    const int n_blocks0 = p.causal ? last_row0 / kTileKV + 1 : p.kv_blocks;
    const int n_blocks = p.causal ? last_row1 / kTileKV + 1 : p.kv_blocks;   // second tile; n_blocks >= n_blocks0
    // The (query tile, key block) pairs in issue order, "uses" u = 0, 1, ...: (0,0), (1,0), (0,1), (1,1), ...
    // and, when the first tile has one block fewer, (1, n_blocks - 1) last.  Use u works in score buffer
    // u % kScoreBufs, on barrier phase (u / kScoreBufs) & 1 of that buffer's barriers.
    constexpr int kBufs = Cfg::kScoreBufs;
    const int n_uses = n_blocks0 + n_blocks;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->q_full), 1);
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(smem_u32(&bars->kv_full[s]), 1);
            mbar_init(smem_u32(&bars->kv_empty[s]), 1);
        }
        for (int b = 0; b < 3; ++b) {
            mbar_init(smem_u32(&bars->s_full[b]), 1);
            for (int h = 0; h < 2; ++h) {
                mbar_init(smem_u32(&bars->p_ready[b][h]), kTileQ);
            }
        }
        for (int w = 0; w < 2; ++w) {
            mbar_init(smem_u32(&bars->pv_done[w]), 1);
        }
        bars->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == kLoadWarp && lane == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
    }
    if (warp == kMmaWarp) {
        tmem_alloc<1>(smem_u32(&bars->tmem_base), kTmemCols);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    // column offsets inside the allocation
    const uint32_t tmem_s0 = tmem_base;                // score buffer b at + b * 128; P (16-bit pairs) reuses its first 64 columns
    const uint32_t tmem_o0 = tmem_base + kBufs * 128;  // O_w at + w * D

    // The softmax keeps a whole row of 128 scores in registers and needs room beside them to overlap
    // the exponentials' latencies; the loader and the issuer need almost none. Whole warpgroups trade.
    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
        if (warp == kLoadWarp) {
        // ---------------------------------------------------------- TMA producer
        if (lane == 0) {
            const uint32_t qf = smem_u32(&bars->q_full);
            mbar_arrive_expect_tx(qf, 2 * Cfg::kTileBytes);
            for (int w = 0; w < 2; ++w) {
                for (int a = 0; a < Cfg::kAtoms; ++a) {
                    tma_load_3d(q_smem + w * Cfg::kTileBytes + a * Cfg::kAtomBytes, &tmap_q, qf, a * 64,
                                q_row0 + w * kTileQ, head);
                }
            }
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = 0; t < 2 * n_blocks && ok; ++t) {  // the second tile's blocks cover the first's
                // tile order: K_0, V_0, K_1, V_1, ...
                const int j = t >> 1;
                const CUtensorMap* map = (t & 1) ? &tmap_v : &tmap_k;
                if (!mbar_wait(smem_u32(&bars->kv_empty[stage]), phase ^ 1u, abort_flag)) {
                    report_timeout(p, abort_flag, 1, stage);
                    ok = false;
                    break;
                }
                const uint32_t full = smem_u32(&bars->kv_full[stage]);
                mbar_arrive_expect_tx(full, Cfg::kTileBytes);
                for (int a = 0; a < Cfg::kAtoms; ++a) {
                    tma_load_3d(kv_smem + stage * Cfg::kTileBytes + a * Cfg::kAtomBytes, map, full, a * 64,
                                j * kTileKV, head);
                }
                if (++stage == (uint32_t)kKvStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the control flow and one elected lane issues. Everything an issue needs
        // (descriptors, tensor-memory and barrier addresses) is then the same in all lanes and can live in
        // uniform registers; issued from inside a one-lane branch each multiply cost the thread about
        // 60 cycles, as long as the tensor core needs to execute it, and the issuer bounded the kernel.
        const bool leader = elect_one();
        constexpr uint32_t idesc_qk = umma_idesc_f16_f32(kTileQ, kTileKV, false, false, kBf16);
        constexpr uint32_t idesc_pv = umma_idesc_f16_f32(kTileQ, D, false, true, kBf16);  // B = V is N-major
        bool ok = true;
        // Descriptor low words: one per operand tile, advanced by compile-time constants per MMA
        // (a 64-wide column block further = +1024, 16 elements along K inside a block = +2,
        // 16 rows further down an N-major V tile = +128, all in units of 16 bytes).
        const uint32_t q_lo0 = desc_lo_kmajor(q_smem);
        auto commit = [&](uint64_t* bar) {
            if (leader) {
                umma_commit<1>(smem_u32(bar));
            }
        };
        // every lane polls; a timeout is reported once
        auto wait = [&](uint64_t* bar, uint32_t parity, uint32_t where) {
            const bool done = mbar_wait(smem_u32(bar), parity, abort_flag);
            if (!done && leader) {
                report_timeout(p, abort_flag, 2, where);
            }
            return __all_sync(0xFFFFFFFFu, done);
        };
        // use u -> (key block j, query tile w); K_j is tile 2j of the ring, V_j tile 2j + 1
        auto use_block = [&](int u, int& j, int& w) {
            if (u < 2 * n_blocks0) {
                j = u >> 1;
                w = u & 1;
            } else {
                j = n_blocks - 1;
                w = 1;
            }
        };
        auto wait_kv = [&](int t, uint32_t& st) {
            st = (uint32_t)(t % kKvStages);
            return wait(&bars->kv_full[st], (uint32_t)((t / kKvStages) & 1), st);
        };
        // S(u) = Q_w K_j^T into score buffer u % kBufs.  (Not split along the keys: with both operands
        // in shared memory a 128 x 64 x 16 step reads 6 KB in 32 cycles, more than shared memory delivers.)
        // (The K tile must have been waited for, and a tcgen05 fence passed, before this is called: the main
        // loop does both before it waits for P, so that nothing stands between the P V issue and this one.
        // A wait and a fence in between cost 3.6 % at head dimension 128.)
        auto issue_qk = [&](int u) {
            int j, w;
            use_block(u, j, w);
            const uint32_t st = (uint32_t)((2 * j) % kKvStages);
            const uint32_t buf = (uint32_t)(u % kBufs);
            const uint32_t k_lo = desc_lo_kmajor(kv_smem + st * Cfg::kTileBytes);
            const uint32_t q_lo = q_lo0 + (uint32_t)w * (Cfg::kTileBytes >> 4);
            if (leader) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (uint32_t)((kk / 4) * (Cfg::kAtomBytes >> 4) + 2 * (kk % 4));
                    umma_f16_ss_cta1(tmem_s0 + buf * 128, q_lo + off, kDescHiSw128, k_lo + off, kDescHiSw128, idesc_qk,
                                     kk != 0 ? 1u : 0u);
                }
                umma_commit<1>(smem_u32(&bars->s_full[buf]));
                if (w == 1) {
                    umma_commit<1>(smem_u32(&bars->kv_empty[st]));  // the second tile is K_j's last reader
                }
            }
        };
        // the K tile of use u has landed
        auto wait_k = [&](int u) {
            int j, w;
            use_block(u, j, w);
            uint32_t st;
            return wait_kv(2 * j, st);
        };
        // O_w (+)= P(u) V_j: A = P in tensor memory (16 keys = 8 packed columns per step), B = the V tile
        // (N-major; its d-halves are one 128-row block apart), in two halves of 64 keys as the softmax
        // hands them over
        auto issue_pv = [&](int u) {
            int j, w;
            use_block(u, j, w);
            uint32_t st;
            // the tile was requested long ago; make sure of it now, while the softmax is still at work
            if (!wait_kv(2 * j + 1, st)) {
                return false;
            }
            const uint32_t buf = (uint32_t)(u % kBufs), parity = (uint32_t)((u / kBufs) & 1);
            const uint32_t v_lo = desc_lo_mnmajor(kv_smem + st * Cfg::kTileBytes, Cfg::kAtomBytes);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (!wait(&bars->p_ready[buf][h], parity, 0x30 + 8 * h + buf)) {
                    return false;
                }
                tcgen05_fence_after();
                if (leader) {
#pragma unroll
                    for (int kk = h * (kTileKV / 32); kk < (h + 1) * (kTileKV / 32); ++kk) {
                        umma_f16_ts_cta1(tmem_o0 + w * D, tmem_s0 + buf * 128 + kk * 8, v_lo + (uint32_t)(kk * 128),
                                         kDescHiSw128, idesc_pv, (j > 0 || kk != 0) ? 1u : 0u);
                    }
                }
            }
            // With three score buffers the softmax of the next block may already be running and may want to
            // rescale O_w: it waits for this.  With two, only the end of the tile matters (a completed
            // s_full of the next block implies this multiply is complete).
            const int n_w = w == 0 ? n_blocks0 : n_blocks;
            if (kBufs == 3 || j == n_w - 1) {
                commit(&bars->pv_done[w]);
            }
            if (w == 1) {
                commit(&bars->kv_empty[st]);  // the second tile is V_j's last reader
            }
            return true;
        };
        do {
            if (!wait(&bars->q_full, 0, 0x20)) {
                break;
            }
            for (int u = 0; u < kBufs && u < n_uses && ok; ++u) {
                ok = wait_k(u);
                if (ok) {
                    tcgen05_fence_after();
                    issue_qk(u);
                }
            }
            // P(u) V, then the score tile that takes over the buffer this multiply frees
            for (int u = 0; u < n_uses && ok; ++u) {
                const bool next_qk = u + kBufs < n_uses;
                // the tiles these multiplies read were requested long ago; make sure of them now, while the
                // softmax is still at work
                if (next_qk && !wait_k(u + kBufs)) {
                    ok = false;
                    break;
                }
                ok = issue_pv(u);
                if (ok && next_qk) {
                    issue_qk(u + kBufs);
                }
            }
        } while (false);
        }
    } else {
        // --------------------------------------------------------------- softmax
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
        const uint32_t w = warp / 4;        // query tile of this warpgroup
        const uint32_t quarter = warp % 4;  // TMEM lanes [32*quarter, +32)
        const uint32_t row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32u) << 16;
        const uint32_t tmem_o = tmem_o0 + w * D + lane_addr;
        const float sl2 = p.scale_log2e;
        float m_ref = -INFINITY;  // row max the stored O and l are relative to (raw scores)
        float l_run = 0.0f;       // running row sum
        bool ok = true;
        const int n_w = w == 0 ? n_blocks0 : n_blocks;  // key blocks of this query tile
        for (int j = 0; j < n_w; ++j) {
            // this (tile, block) pair's place in the issue order, hence its score buffer and barrier phase
            const int u = w == 0 ? 2 * j : 2 * j + (j < n_blocks0 ? 1 : 0);
            const uint32_t buf = (uint32_t)(u % kBufs), parity = (uint32_t)((u / kBufs) & 1);
            const uint32_t tmem_s = tmem_s0 + buf * 128 + lane_addr;
            if (!mbar_wait(smem_u32(&bars->s_full[buf]), parity, abort_flag, kSoftmaxBackoffNs)) {
                if (lane == 0) {
                    report_timeout(p, abort_flag, 3, 0x10 + buf);
                }
                ok = false;
                break;
            }
            // With two score buffers a completed s_full also means every earlier MMA of the issuing thread is
            // complete: P_w of the previous block has been consumed and O_w is not being written.  With three
            // the previous block's P V may still be running; whoever rescales O_w waits for it below.
            tcgen05_fence_after();
            uint32_t r[128];
            {
                uint32_t(&r0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[0]);
                uint32_t(&r1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[32]);
                uint32_t(&r2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[64]);
                uint32_t(&r3)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[96]);
                tmem_ld_32x32b_x32(tmem_s, r0);
                tmem_ld_32x32b_x32(tmem_s + 32, r1);
                tmem_ld_32x32b_x32(tmem_s + 64, r2);
                tmem_ld_32x32b_x32(tmem_s + 96, r3);
                tmem_ld_wait();
            }
            int valid = p.S - j * kTileKV;  // keys of this block that exist
            bool masked = valid < kTileKV;  // uniform over the CTA
            if (p.causal) {
                // keys of this block this row may see: global key index <= global query index
                const int row_global = q_row0 + (int)w * kTileQ + (int)row;
                const int seen = row_global - j * kTileKV + 1;
                valid = seen < valid ? seen : valid;
                masked = masked || (j + 1) * kTileKV > q_row0 + (int)w * kTileQ + 1;  // uniform over the tile
            }
            if (masked) {
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    if (i >= valid) {
                        r[i] = 0xFF800000u;  // -inf
                    }
                }
            }
            // four independent chains of three-input max
            float m4[4] = {__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]),
                           __uint_as_float(r[3])};
#pragma unroll
            for (int i = 4; i < 124; i += 8) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    m4[c] = max3(m4[c], __uint_as_float(r[i + 2 * c]), __uint_as_float(r[i + 2 * c + 1]));
                }
            }
            m4[0] = max3(m4[0], __uint_as_float(r[124]), __uint_as_float(r[125]));
            m4[1] = max3(m4[1], __uint_as_float(r[126]), __uint_as_float(r[127]));
            const float m_blk = fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]);
            // Lazy rescale: keep the old reference max unless the new one is more than 2^8 above it.
            const bool grow = j == 0 || (m_blk - m_ref) * sl2 > kRescaleThreshold;
            float alpha = 1.0f;
            if (grow) {
                alpha = ex2_approx((m_ref - m_blk) * sl2);  // 0 on the first block
                m_ref = m_blk;
            }
            // Rescale O_w when some row of this warp moved its reference max (never on the first block).
            // It has to be finished before the first half of P is handed over: from then on the issuer
            // accumulates into O_w.
            if (j > 0 && __any_sync(0xFFFFFFFFu, grow)) {
                if (kBufs == 3) {
                    // O_w must have taken the previous block's P V before it is rescaled.  That multiply is the
                    // j-th completion of pv_done[w] (this block's cannot be issued before this thread hands P
                    // over), so the barrier has completed j - 1 or j phases: wait for parity (j - 1) & 1.
                    if (!mbar_wait(smem_u32(&bars->pv_done[w]), (uint32_t)((j - 1) & 1), abort_flag)) {
                        if (lane == 0) {
                            report_timeout(p, abort_flag, 3, 0x18 + w);
                        }
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                }
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32b_x32(tmem_o + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    }
                    tmem_st_32x32b_x32(tmem_o + c * 32, o);
                }
            }
            const float neg_m = -m_ref * sl2;
            const float ks = sl2 * (1.0f / 64.0f);
            const float cs = (neg_m + kPolyLo) * (1.0f / 64.0f);
            // packed forms where both elements of a pair take the same step: half the issue slots
            const uint64_t sl2_2 = pack2(sl2, sl2);
            const uint64_t neg_m2 = pack2(neg_m, neg_m);
            uint64_t l_blk2 = pack2(0.0f, 0.0f);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t packed[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float s0 = __uint_as_float(r[half * 64 + 2 * i]);
                    const float s1 = __uint_as_float(r[half * 64 + 2 * i + 1]);
                    float p0, p1;
                    if ((i & 7) < kPolyPairs<D>) {
                        ex2_poly2(s0, s1, ks, cs, p0, p1);
                    } else {
                        float x0, x1;
                        unpack2(fma2(pack2(s0, s1), sl2_2, neg_m2), x0, x1);
                        p0 = ex2_approx(x0);
                        p1 = ex2_approx(x1);
                    }
                    l_blk2 = add2(l_blk2, pack2(p0, p1));
                    packed[i] = pack_half2<kBf16>(p0, p1);
                }
                tmem_st_32x32b_x32(tmem_s + half * 32, packed);
                // hand this half of P_w over: the issuer multiplies it while the other half is computed
                tmem_st_wait();
                tcgen05_fence_before();
                mbar_arrive(smem_u32(&bars->p_ready[buf][half]));
            }
            float l_blk0, l_blk1;
            unpack2(l_blk2, l_blk0, l_blk1);
            l_run = l_run * alpha + (l_blk0 + l_blk1);
        }
        // ---- epilogue: O_w / l -> fp16 -> global
        if (ok) {
            // two score buffers: pv_done[w] completes once, at the end; three: once per block
            if (!mbar_wait(smem_u32(&bars->pv_done[w]), kBufs == 3 ? (uint32_t)((n_w - 1) & 1) : 0u, abort_flag, 20)) {
                if (lane == 0) {
                    report_timeout(p, abort_flag, 3, 0x28 + w);
                }
                ok = false;
            }
        }
        if (ok) {
            tcgen05_fence_after();
            const float inv_l = 1.0f / l_run;
            const int q_row = q_row0 + (int)w * kTileQ + (int)row;
            uint16_t* dst = static_cast<uint16_t*>(p.o) + ((size_t)head * p.S + (size_t)(q_row < p.S ? q_row : 0)) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_o + c * 32, r);
                tmem_ld_wait();
                if (q_row < p.S) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 v;
                        v.x = pack_half2<kBf16>(__uint_as_float(r[8 * q4 + 0]) * inv_l, __uint_as_float(r[8 * q4 + 1]) * inv_l);
                        v.y = pack_half2<kBf16>(__uint_as_float(r[8 * q4 + 2]) * inv_l, __uint_as_float(r[8 * q4 + 3]) * inv_l);
                        v.z = pack_half2<kBf16>(__uint_as_float(r[8 * q4 + 4]) * inv_l, __uint_as_float(r[8 * q4 + 5]) * inv_l);
                        v.w = pack_half2<kBf16>(__uint_as_float(r[8 * q4 + 6]) * inv_l, __uint_as_float(r[8 * q4 + 7]) * inv_l);
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = v;
                    }
                }
            }
        }
    }

    // ----------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
        probe[2] = (unsigned long long)clock64();
        probe[3] = global_timer_ns();
    }
}

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

// [BH][S][D] fp16 tensor, boxes of 128 rows x 64 columns (128 bytes, swizzled) of one head.
static int make_tmap_bsd(CUtensorMap* map, const void* base, int BH, int S, int D, bool bf16)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        return SPORK_ERR_DRIVER;
    }
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)BH};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)S * D * 2};
    const cuuint32_t box[3] = {64, 128, 1};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                          elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : SPORK_ERR_DRIVER;
}

// Head dimension 128 runs the two-buffer kernel, head dimension 64 the rotating-buffer kernel (only the
// pairs in use are instantiated).
template <int D, bool kBf16>
struct KernelFor {
    static auto get(bool) { return attn_fwd_kernel<D, kBf16>; }
};
template <bool kBf16>
struct KernelFor<128, kBf16> {
    static auto get(bool causal)
    {
        return causal ? attn_fwd_two_kernel<128, kBf16, true> : attn_fwd_two_kernel<128, kBf16, false>;
    }
};

template <int D, bool kBf16>
static int launch(int BH, int S, const void* q, const void* k, const void* v, void* o, float scale, bool causal,
                  DeviceState& dev, cudaStream_t stream)
{
    using Cfg = Config<D>;
    auto kernel = KernelFor<D, kBf16>::get(causal);
    static std::once_flag attr_once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(attr_once[dev.ordinal], [&] {
        attr_err[dev.ordinal] = cudaFuncSetAttribute(KernelFor<D, kBf16>::get(false),
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (attr_err[dev.ordinal] == cudaSuccess) {
            attr_err[dev.ordinal] = cudaFuncSetAttribute(
                KernelFor<D, kBf16>::get(true), cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        }
    });
    if (attr_err[dev.ordinal] != cudaSuccess) {
        return (int)attr_err[dev.ordinal];
    }
    Params p{};
    p.BH = BH;
    p.S = S;
    p.D = D;
    p.q_pairs = (S + 2 * kTileQ - 1) / (2 * kTileQ);
    p.kv_blocks = (S + kTileKV - 1) / kTileKV;
    p.causal = causal ? 1 : 0;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.o = o;
    p.status = dev.status_word;
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tmap_bsd(&tq, q, BH, S, D, kBf16)) != 0 || (rc = make_tmap_bsd(&tk, k, BH, S, D, kBf16)) != 0 ||
        (rc = make_tmap_bsd(&tv, v, BH, S, D, kBf16)) != 0) {
        return rc;
    }
    const long long ctas = (long long)BH * p.q_pairs;
    if (ctas > 0x7FFFFFFFll) {
        return SPORK_ERR_TOO_LARGE;
    }
    kernel<<<(unsigned)ctas, kNumThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, p);
    return (int)cudaGetLastError();
}

__global__ void f32_to_f16_kernel(const float* src, __half* dst, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        dst[i] = __float2half_rn(src[i]);
    }
}

__global__ void f16_to_f32_kernel(const __half* src, float* dst, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        dst[i] = __half2float(src[i]);
    }
}

}  // namespace attn_sm100
}  // namespace spork

extern "C" int spork_attn_sm100_supports(int BH, int S, int D)
{
    return (BH >= 0 && S >= 0 && (D == 64 || D == 128)) ? 1 : 0;
}

static int attn_dispatch(int BH, int S, int D, const void* q, const void* k, const void* v, void* o, float scale,
                         void* stream, bool bf16, bool causal = false)
{
    if (!spork_attn_sm100_supports(BH, S, D)) {
        return SPORK_ERR_UNSUPPORTED_SHAPE;
    }
    if (BH == 0 || S == 0) {
        return 0;
    }
    auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
    // scale must be positive: the kernel folds it into the exponent ((s - max) * scale * log2 e), and with
    // scale = 0 the -inf of a masked score would meet a zero factor (NaN).  Negative or NaN scales are
    // refused as well.
    if (!q || !k || !v || !o || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !(scale > 0.0f)) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    spork::DeviceState* dev = nullptr;
    const int rc = spork::current_device_state(&dev);
    if (rc) {
        return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    using namespace spork::attn_sm100;
    if (D == 64) {
        return bf16 ? launch<64, true>(BH, S, q, k, v, o, scale, causal, *dev, s)
                    : launch<64, false>(BH, S, q, k, v, o, scale, causal, *dev, s);
    }
    return bf16 ? launch<128, true>(BH, S, q, k, v, o, scale, causal, *dev, s)
                : launch<128, false>(BH, S, q, k, v, o, scale, causal, *dev, s);
}

extern "C" int spork_attn_sm100_fwd_ex(int BH, int S, int D, const void* q, const void* k, const void* v, void* o,
                                       float scale, int bf16, int causal, void* stream)
{
    return attn_dispatch(BH, S, D, q, k, v, o, scale, stream, bf16 != 0, causal != 0);
}

extern "C" int spork_attn_sm100_fwd_f16(int BH, int S, int D, const void* q, const void* k, const void* v, void* o,
                                        float scale, void* stream)
{
    return attn_dispatch(BH, S, D, q, k, v, o, scale, stream, false);
}

extern "C" int spork_attn_sm100_fwd_bf16(int BH, int S, int D, const void* q, const void* k, const void* v, void* o,
                                         float scale, void* stream)
{
    return attn_dispatch(BH, S, D, q, k, v, o, scale, stream, true);
}

// Same signature and meaning as the reference's htod_f32_tk_4090_fwd
// (tk_4090_fwd.hpp:7): host fp32 (N, d) matrices in, host fp32 out, one head,
// scale 1/sqrt(d).  Inputs are rounded to fp16 on the device.  On failure the
// output is filled with NaN and a message goes to stderr (the reference's
// entry point returns void as well).
extern "C" void htod_f32_attn_sm100_fwd(int N, int d, const float* q, const float* k, const float* v, float* o)
{
    using namespace spork::attn_sm100;
    auto fail = [&](const char* what, int code) {
        fprintf(stderr, "htod_f32_attn_sm100_fwd: %s (code %d)\n", what, code);
        if (o && N > 0 && d > 0) {
            for (size_t i = 0; i < (size_t)N * d; ++i) {
                o[i] = NAN;
            }
        }
    };
    if (N <= 0 || d <= 0) {
        return;
    }
    if (!q || !k || !v || !o || !spork_attn_sm100_supports(1, N, d)) {
        fail("unsupported shape or null pointer (d must be 64 or 128)", SPORK_ERR_UNSUPPORTED_SHAPE);
        return;
    }
    spork::DeviceState* dev = nullptr;
    int rc = spork::current_device_state(&dev);
    if (rc) {
        fail("no usable device", rc);
        return;
    }
    const size_t n = (size_t)N * d;
    // slot 0: fp32 staging (n floats), slot 1: q,k,v,o fp16 (4n halves)
    if ((rc = spork::ensure_staging(*dev, 0, n * sizeof(float))) != 0 ||
        (rc = spork::ensure_staging(*dev, 1, 4 * n * sizeof(__half) + 64)) != 0) {
        fail("staging allocation", rc);
        return;
    }
    cudaStream_t s = cudaStreamPerThread;
    float* f32 = static_cast<float*>(dev->staging[0]);
    __half* h = static_cast<__half*>(dev->staging[1]);
    const size_t n_pad = (n + 7) & ~size_t(7);  // keeps every fp16 matrix 16-byte aligned
    const float* src[3] = {q, k, v};
    const unsigned blocks = (unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < 3 && e == cudaSuccess; ++i) {
        e = cudaMemcpyAsync(f32, src[i], n * sizeof(float), cudaMemcpyHostToDevice, s);
        f32_to_f16_kernel<<<blocks, 256, 0, s>>>(f32, h + i * n_pad, n);
    }
    if (e != cudaSuccess) {
        fail("copy to device", (int)e);
        return;
    }
    rc = spork_attn_sm100_fwd_f16(1, N, d, h, h + n_pad, h + 2 * n_pad, h + 3 * n_pad, 1.0f / sqrtf((float)d), s);
    if (rc) {
        fail("launch", rc);
        return;
    }
    f16_to_f32_kernel<<<blocks, 256, 0, s>>>(h + 3 * n_pad, f32, n);
    e = cudaMemcpyAsync(o, f32, n * sizeof(float), cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) {
        fail("copy to host", (int)e);
        return;
    }
    rc = spork_gemm_sm100_status(s, nullptr);
    if (rc) {
        fail("device status", rc);
    }
}
