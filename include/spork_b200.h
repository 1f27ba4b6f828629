/* C ABI of libspork_b200: hand-written sm_100a (B200) kernels behind the launch
 * interface of the akeley98/spork GEMM/attention testbed.
 *
 * Conventions shared by every entry point (they mirror the reference's launch
 * functions, gemm/gemm_sm90.h:14, gemm/gemm_sm80.h:5-6, gemm/gemm_baseline.h:5):
 *   - the caller owns every buffer; pointers are DEVICE pointers unless the
 *     name says "htod" (host in, host out);
 *   - launches are asynchronous on the caller's stream and never synchronise;
 *   - `stream` is a cudaStream_t passed as void* so that this header needs no
 *     CUDA include;
 *   - return value 0 = success; a positive value below 10000 is a cudaError_t;
 *     values >= SPORK_ERR_BASE are this library's own codes (below).
 * Unlike the reference (which asserts and prints), argument errors are
 * returned, never trapped.
 */
#ifndef SPORK_B200_H
#define SPORK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Every entry point is exported; everything else in the library is hidden. */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define SPORK_ERR_BASE 10000
#define SPORK_ERR_BAD_ARGUMENT 10001   /* null / misaligned pointer, unknown variant */
#define SPORK_ERR_UNSUPPORTED_SHAPE 10002 /* see spork_gemm_sm100_supports */
#define SPORK_ERR_NO_SM100 10003       /* current device is not compute capability 10.x */
#define SPORK_ERR_DRIVER 10004         /* tensor-map encode or driver entry point failed */
#define SPORK_ERR_DEVICE_TIMEOUT 10005 /* a bounded device-side wait ran out (status word set) */
#define SPORK_ERR_TOO_LARGE 10006      /* beyond a stated fixed capacity */
#define SPORK_ERR_DEVICE_CHECK 10007   /* debug build (-DSPORK_CHECKED): a device-side range check failed (status word set) */

/* ---- GEMM: C[M,N] (fp32, row-major) = A[M,K] (fp16, row-major) . B[N,K]^T (fp16, row-major) ----
 * Operand layout of the reference harness's hot call
 * `GPU_Tensors{M,N,K,d_a,d_bCol,d_c,0,1,0}` (gemm/gemm_test.cu:305,365), with
 * fp16 inputs and fp32 accumulation/output instead of fp32/TF32. */

/* 1 if (M,N,K) can be launched: K % 8 == 0 (a row of A or B must be a multiple
 * of 16 bytes for TMA), everything else arbitrary (ragged M, N, K are
 * handled; M, N or K == 0 is legal).  Replaces matmul_sm80_supports
 * (gemm/gemm_sm80.h:6) / the asserts of gemm/gemm_sm90.cu:1269-1276. */
int spork_gemm_sm100_supports(uint32_t M, uint32_t N, uint32_t K);

/* Launch.  variant: 0 = choose (width from N, CTA pairs; single CTAs with
 * tiles at most 128 wide for small latency-bound problems; 256 x 512 tiles per
 * CTA pair for large problems with K >= 4096), 64 / 128 / 256 / 512 =
 * width of the output tile along N, taken literally, on CTA pairs (the
 * n64/n128/n256 variants of xgemm_Sm90_n{64,128,256}.py; 512 has no counterpart).
 * Replaces matmul_sm90(t, gemm_sm90_k_mode::output_stationary, stream)
 * (gemm/gemm_sm90.cu:1344-1360). */
int spork_gemm_sm100_f16f32(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C, int variant,
                            void* stream);

/* The same kernel on the reference's own operand type: fp32 A and B read as tf32
 * by the tensor cores (tcgen05.mma.kind::tf32), fp32 accumulation and output -
 * what matmul_sm90 / matmul_sm80 / cublasSgemm-in-TF32-mode compute
 * (gemm/gemm_sm90.cu:555-614, gemm/gemm_sm80.cu:92-101, gemm/gemm_test.cu:208).
 * Same layout (A MxK, B NxK, C MxN, all row-major); K % 4 == 0.  split_k >= 1
 * as in the _ex entry point. */
int spork_gemm_sm100_tf32f32(uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B, float* C,
                             int variant, int split_k, void* stream);

/* Launch with every tunable explicit (benchmark sweeps and tests).
 *   block_n   64 / 128 / 256   output-tile width
 *   cta_group 1 = one CTA per tile (128 x block_n),
 *             2 = a CTA pair per tile (256 x block_n, tcgen05 cta_group::2),
 *             0 = the tile is left to the library as in spork_gemm_sm100_f16f32
 *             (block_n is then its `variant`, 0 allowed); with split_k = 0 this
 *             is the fully automatic launch
 *   split_k   0: chosen by the library: 1, or, for a problem with fewer 256-wide
 *             output tiles than CTA pairs and a long K, the count that fills
 *             the waves best, or stream-K (-1) when the last of several waves
 *             of tiles is less than half full (see spork_gemm_sm100_plan and
 *             spork_gemm_sm100_choice);
 *             >= 1: K is cut into split_k ranges whose partial products are
 *             added into C with TMA reduce-add (C is zeroed first); the
 *             counterpart of gemm_sm90_k_mode::split_k_outer
 *             (gemm/gemm_sm90.h:8, gemm/gemm_sm90.cu:1096-1114).
 *             -1: stream-K, the counterpart of gemm_sm90_k_mode::stream_k_*
 *             (gemm/gemm_sm90.h:10-11, gemm/gemm_sm90.cu:1004-1094): whole
 *             waves of tiles run one tile per CTA pair; each tile of the last
 *             partial wave, when that wave is at most half full, is cut into
 *             as many equal K ranges as there are CTA pairs to run them at the
 *             same time, all tiles at the same K offsets (so concurrent pairs
 *             still sweep shared strips of A and B through L2), and the ranges
 *             are reduce-added into C.  The kernel zeroes those tiles itself
 *             while its epilogue warps wait for the first tile, and its CTAs
 *             meet at a device counter before the first reduce-add (a bounded
 *             wait; the last CTA to leave resets the counter, so a launch can
 *             be replayed from a CUDA graph): the launch relies on all its CTAs being resident
 *             together, which holds when it has the device to itself, so do
 *             not run stream-K launches of several streams at the same time.
 *             A last wave more than half full runs whole (no ranges).
 *             <= -2: |split_k| ranges like >= 2, but the ranges of one tile are
 *             neighbours in the schedule (K fastest), the counterpart of
 *             gemm_sm90_k_mode::split_k_inner (gemm/gemm_sm90.h:9).
 *   block_n   also 512: 256 x 512 tiles per CTA pair (cta_group 2, split_k >= 0
 *             or <= -2), the tile the library picks by itself for large
 *             compute-bound problems with K >= 4096.
 *   max_ctas  0 = one CTA per SM, else an upper bound on the grid. */
int spork_gemm_sm100_f16f32_ex(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C,
                               int block_n, int cta_group, int split_k, int max_ctas, void* stream);

/* A batch of L independent products in one launch: C[l] = A[l] * B[l]^T with
 * A [L][M][K], B [L][N][K] (fp16) and C [L][M][N] (fp32) each stored as L
 * contiguous row-major matrices.  The counterpart of the batch dimension `L` of
 * the reference's generated entry points (xgemm_Sm90.py:45-48, C: f32[L,N,M];
 * call sites gemm/gemm_test.cu:310-362 pass L = 1); a caller with that
 * column-major C swaps the operands, as for the single product.  The kernel is
 * the same persistent kernel: the batch index is one more coordinate of the tile
 * scheduler and of 3-D tensor maps, so ragged M and N are zero-filled and
 * clipped per matrix.  `variant` as for spork_gemm_sm100_f16f32; split_k >= 0 as
 * for the _ex form (no stream-K over a batch).  L = 0 is a no-op. */
int spork_gemm_sm100_f16f32_batched(uint32_t L, uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B,
                                    float* C, int variant, int split_k, void* stream);

/* Allocation-free GEMM.  Has no counterpart in the reference (whose harness
 * allocates freely, gemm/gemm_test.cu:218-226).  For callers that cannot
 * allocate device memory at call time: code living inside an arena that already
 * owns the GPU's memory, processes that lock their allocator after start-up,
 * latency paths that cannot afford cudaMalloc's implicit synchronisation.
 * Same product as spork_gemm_sm100_f16f32, computed as `split_k` (>= 1) partial
 * products over ranges of K that are summed in a fixed order (bit-reproducible).
 * All scratch (status word + split-K workspace) is a fixed 64 MiB array inside
 * the library image, held by every GPU that loads the library until exit:
 *   - split_k * M * ceil4(N) * 4 bytes must be <= 64 MiB, else SPORK_ERR_TOO_LARGE;
 *   - the first call on a device resolves the array's device address and sets
 *     kernel attributes: make it before any stream capture;
 *   - calls on one device share the array: calls that may overlap on the GPU
 *     race and must be serialised by the caller;
 *   - M = N = K = 0 queries: synchronises `stream`, returns and clears
 *     SPORK_ERR_DEVICE_TIMEOUT if a launch of this entry point gave up a wait.
 * Calls no cudaMalloc / cudaFree / allocating library routine. */
int spork_gemm_sm100_f16f32_static(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C,
                                   int split_k, void* stream);

/* SM clock (MHz) the most recent GEMM or attention launch on the current device
 * really ran at: one CTA (the first of a GEMM, which lives as long as the launch;
 * the last of an attention launch) notes SM cycles and wall-clock time at both
 * ends of its life.  Synchronises `stream`.  Under the power cap this is far below
 * the nominal clock that the management library reports.  No counterpart in the
 * reference. */
int spork_gemm_sm100_last_clock_mhz(void* stream, double* mhz);

/* Process-wide tuning of later launches (benchmark sweeps; the defaults are the
 * measured best).  stages: shared-memory ring depth, 0 = as deep as fits;
 * group_m: m-tiles per raster group, 0 = default; l2_hints, low four bits: 0 =
 * default (A and B loads evict-last), bit 0 = A loads evict-last, bit 1 = B loads
 * evict-last, bit 2 = B loads evict-first, 8 = no hints at all;
 * backoff_ns: sleep between polls of the long waits, 0 = spin.  Bits 8..9 of
 * l2_hints: 128-byte column blocks per ring stage (1 or 2; 0 = chosen per shape:
 * 2 for skinny HBM-bound problems).  Bits 4..6 of
 * l2_hints switch diagnostic experiments whose RESULTS ARE UNDEFINED (0x10 the
 * epilogue drops its stores, 0x20 the producer stops loading after the first
 * ring fill, 0x40 stores go straight from registers).  Bits 10..11: 256 x 512
 * tiles per CTA pair for problems whose tile is left to the library (0 = chosen
 * per shape, 1 = never, 2 = always); bits 12..15: K blocks by which one half of
 * such a tile runs ahead of the other at the tile's ends (0 = default);
 * bits 16..23: their raster group (0 = default); bit 24: launches are plain
 * stream-ordered kernels instead of programmatic dependents (by default a launch
 * sets up its barriers and tensor memory while the previous kernel in the stream
 * is still finishing on other SMs, and waits for it before touching global
 * memory); bit 25: problems that underfill the machine keep 256-wide tiles (by
 * default variant 0 narrows the tile to 128 or 64 columns when that fills the
 * waves better).  spork_gemm_sm100_tuning reads
 * the knobs back.  The reference
 * fixes the equivalent choices at compile time (gemm/gemm_sm90.cu:1278-1289). */
int spork_gemm_sm100_tune(int stages, int group_m, int l2_hints, int backoff_ns);

/* Host-side model of the kernels' barrier protocol (no GPU, no CUDA call): runs
 * the roles of CTA group `group` of the launch plan of (M, N, K, block_n,
 * cta_group, split_k >= 1 or -1, max_ctas, sm_count) - producers, TMA engines,
 * MMA issuer, tensor pipe, epilogue warps - as cooperative agents over modelled
 * mbarriers, in an interleaving drawn from `seed`, with a ring of `stages` stages
 * and (block_n = 512) the given skew.  Returns 0 if every invariant held, else
 * 1 = deadlock, 2 = a stage was refilled before it was read, 3 = an MMA read a
 * stage that did not hold its K block, 4 = an MMA wrote an accumulator the
 * epilogue still read, 5 = the epilogue read an accumulator that was not final,
 * 6 = an output part was not written exactly once.  `inject` plants a protocol bug to show the checks notice:
 * 1 = (block_n 512) a stage is released after the first half read it, 2 = the
 * issuer does not wait for the accumulator, 3 = the producer does not wait for
 * the stage; 0 = none.  stats (optional, 4 values): work items, MMA operations
 * executed, scheduling steps, CTA groups of the plan.  Stands in for the race
 * checker that the reference's development relies on (compute-sanitizer). */
int spork_gemm_sm100_ring_model(uint32_t M, uint32_t N, uint32_t K, int block_n, int cta_group, int split_k,
                                int max_ctas, int sm_count, int stages, int skew, uint32_t seed, uint32_t group,
                                int inject, uint64_t* stats);

/* What spork_gemm_sm100_f16f32(M, N, K, ..., variant, ...) (split_k = 1) or the
 * _ex entry (another split_k) resolves to on a device with `sm_count` SMs, without
 * launching anything: out[0] = tile width (64 / 128 / 256, or 512 = the 256 x 512
 * pair-tile kernel), out[1] = CTAs per tile, out[2] = 128-byte column blocks per
 * ring stage, out[3] = K split (-1 = stream-K).  Pure arithmetic (no CUDA call).
 * The reference fixes these choices at compile time
 * (gemm/gemm_sm90.cu:1278-1289). */
int spork_gemm_sm100_choice(uint32_t M, uint32_t N, uint32_t K, int variant, int split_k, int sm_count, int tf32,
                            int* out);

/* Every GEMM launch needs three TMA descriptors (tensor maps).  They are encoded
 * by the driver once per (base address, shape, tile box, element type) and host
 * thread and reused by later launches on the same operands; this returns how many
 * look-ups of the process hit and missed that cache.  The reference encodes them
 * on every launch (gemm/gemm_sm90.cu:1167-1206). */
int spork_gemm_sm100_tmap_cache_stats(uint64_t* hits, uint64_t* misses);

/* The counter pairs stream-K launches meet at, read back after `stream` has
 * drained: out[32] = (warps that zeroed their share, CTAs that left) of each of
 * the 16 pairs.  Every pair is back at zero whenever no stream-K launch is in
 * flight: the last CTA to leave resets it, which is what makes the value a launch
 * waits for independent of earlier launches.  Diagnostic; no counterpart in the
 * reference. */
int spork_gemm_sm100_stream_k_counters(uint32_t* out, void* stream);

/* Tracing of the 256 x 512 kernel: later launches make their first CTA write SM
 * clock stamps (clock64) of its tile hand-overs into `device_buffer`, eight
 * 64-bit values per work item of that CTA, for the first `items` work items:
 * [0], [1] the issuer found accumulator half 0 / 1 free; [2], [3], [4] half 0 was
 * final, sat in the epilogue's registers, had its last store issued; [5], [6], [7]
 * the same for half 1.  The buffer must stay valid until tracing is switched off
 * with (NULL, 0).  Process-wide, like the tuning knobs.  No counterpart in the
 * reference (its tracing is nvtx ranges and event timing, gemm/gemm_test.cu). */
int spork_gemm_sm100_trace(void* device_buffer, uint32_t items);

/* The knobs as later launches will see them: out[0] = ring depth, [1] = raster
 * group, [2] = the L2 hint bits a launch carries (bit 0 = A evict-last, bit 1 = B
 * evict-last, bit 2 = B evict-first; 0 = none), [3] = poll back-off, [4] =
 * experiment bits, [5] = column blocks per stage, [6] = 256 x 512 tile choice,
 * [7] = its skew, [8] = its raster group, [9] = 1 if launches are not programmatic
 * dependents.  capacity >= 10.  No counterpart in the reference. */
int spork_gemm_sm100_tuning(int* out, int capacity);

/* Host-only view of how a launch would be laid out (no CUDA call; usable without a
 * GPU).  Arguments as for the _ex entry point, plus the SM count to plan for and
 * tf32 (0/1).  out[10] = tiles_m, tiles_n, K blocks, splits, K blocks per split,
 * CTA groups (CTAs / cta_group), whole-tile count, stream-K tile count, K blocks
 * per stream-K range, ranges per stream-K tile.  split_k = 0 resolves the split
 * count only (stream-K is chosen in spork_gemm_sm100_choice).  The reference computes the
 * equivalent inside its kernel (gemm/gemm_sm90.cu:1004-1129). */
int spork_gemm_sm100_plan(uint32_t M, uint32_t N, uint32_t K, int block_n, int cta_group, int split_k, int max_ctas,
                          int sm_count, int tf32, uint32_t* out);

/* The work items CTA group `group` would process, in order: 5 words per item
 * (m_tile, n_tile, first K block, end K block, 1 if the partial tile is added
 * into C).  Returns the item count (items beyond `capacity` are not written),
 * or -1 on bad arguments. */
int spork_gemm_sm100_plan_items(uint32_t M, uint32_t N, uint32_t K, int block_n, int cta_group, int split_k,
                                int max_ctas, int sm_count, int tf32, uint32_t group, uint32_t* out,
                                uint32_t capacity);

/* Synchronises `stream`, then returns and clears the device status word of the
 * current device: 0, or SPORK_ERR_DEVICE_TIMEOUT if a kernel abandoned a
 * bounded wait (detail word through *detail when non-null).  Replaces the
 * reference's cudaGetLastError polling (gemm/gemm_test.cu:474-477). */
int spork_gemm_sm100_status(void* stream, uint32_t* detail);

/* Self-test of the failure-detection path: launches a one-warp kernel that waits,
 * with the library's bounded wait, on a barrier nothing arrives on.  After
 * `limit_us` microseconds (1 .. 1,000,000) the wait gives up, the kernel sets the
 * device status word and returns; the next spork_gemm_sm100_status call then
 * reports SPORK_ERR_DEVICE_TIMEOUT and the context stays usable.  The reference
 * spins without bound (gemm/gemm_sm90.cu:434-440) and has no such path. */
int spork_selftest_bounded_wait(uint32_t limit_us, void* stream);

/* Self-test of the debug build's range checks (libspork_b200_checked.so, built with
 * -DSPORK_CHECKED: the kernels test every shared-memory and tensor-memory address
 * and every TMA coordinate against what they allocated, record the first failure
 * in the status word and skip the access).  which = 0 / 1 / 2 asks the checks
 * about a shared-memory range, a tensor-memory column range or a TMA coordinate
 * that is out of bounds - nothing is accessed - so that the next
 * spork_gemm_sm100_status reports SPORK_ERR_DEVICE_CHECK with detail
 * 0xC0000000 | (0x701 + which) << 16; which = 3 asks three legal questions and
 * leaves the word clear.  In the normal build: SPORK_ERR_UNSUPPORTED_SHAPE.  The
 * reference's counterpart is DEVICE_ASSERT (gemm/gemm_sm90.cu:15), a trap. */
int spork_selftest_range_check(int which, void* stream);

/* Host-buffer convenience (the htod_f32_* pattern of tk_4090_fwd.hpp:7): copies
 * A and B to the device, runs the GEMM, copies C back and synchronises.  A and B
 * arrive in alternating row chunks on a copy-in stream; each arrival makes a
 * strip of C computable, which is multiplied on a compute stream and copied
 * back on a copy-out stream, so both directions of the host link and the GEMMs
 * overlap (pass pinned host memory for that; pageable memory works,
 * serialised).  Device staging buffers,
 * streams and events are created on first use and kept. */
int spork_gemm_sm100_htod_f16f32(uint32_t M, uint32_t N, uint32_t K, const void* hA, const void* hB, float* hC);

/* ---- Harness kernels (gemm/gemm_test.cu) --------------------------------- */

/* Seeded fixture fill of a rows x cols fp16 matrix; code: 0 sparse random,
 * 1 identity, 2 tiled numbers (gemm/gemm_test.cu:55-96), 3 uniform [-1,1),
 * 4 unit normal as a sum of twelve hashed uniforms (bit-reproducible on the
 * host, tails end at +-6), 5 unit normal by Box-Muller (true tails; the host
 * generator agrees statistically, not bit for bit).  transpose_rule as in the
 * reference. */
int spork_init_test_data_f16(void* d_tensor, uint32_t rows, uint32_t cols, int code, uint32_t seed,
                             int transpose_rule, void* stream);

/* Same fill for a window of a larger logical matrix: element (r, c) of the
 * buffer takes the value of element (row0 + r, col0 + c).  A rank of an
 * M-sharded run fills its own slab of A this way; the reference is single-GPU
 * (gemm/gemm_main.cpp:10) and always fills whole matrices. */
int spork_init_test_data_f16_at(void* d_tensor, uint32_t rows, uint32_t cols, int code, uint32_t seed,
                                int transpose_rule, uint32_t row0, uint32_t col0, void* stream);

/* The reference's oracle kernel restated for fp16 inputs: fp32 FFMA, k
 * ascending (gemm/gemm_baseline.cu:19-168).  Same operand layout as above. */
int spork_gemm_baseline_f16f32(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C,
                               void* stream);

/* Element-wise comparison of two rows x cols fp32 matrices on the device.
 * out[0] = packed (row << 32 | col) of the first element failing the
 * reference's sign + ratio rule (gemm/gemm_test.cu:131-154), UINT64_MAX if
 * none; out[1] = bit pattern of max |a - b| as a double.  `d_out` is a device
 * buffer of two uint64. */
int spork_compare_f32(const float* d_a, const float* d_b, uint32_t rows, uint32_t cols, uint64_t* d_out,
                      void* stream);

/* ---- Attention forward ---------------------------------------------------
 * O = softmax(Q K^T * scale) V per head; q, k, v, o are [BH][S][D] fp16,
 * row-major, each head laid out like the reference's single (N, d) problem
 * (matrix_util.hpp:40-45); softmax in fp32.  D is 64 or 128; scale must be
 * positive (simple_attn's default is 1 / sqrt(D), torch_attn.py:11-16; zero,
 * negative and NaN are refused with SPORK_ERR_BAD_ARGUMENT).  Replaces
 * launch_tk_4090_fwd_kernel (tk_4090_fwd.hpp:5). */
int spork_attn_sm100_supports(int BH, int S, int D);
int spork_attn_sm100_fwd_f16(int BH, int S, int D, const void* q, const void* k, const void* v, void* o, float scale,
                             void* stream);
/* Same with bfloat16 q, k, v, o: the element type of the reference's HostAttnArgs
 * (matrix_util.hpp:40-45) and of launch_tk_4090_fwd_kernel's output. */
int spork_attn_sm100_fwd_bf16(int BH, int S, int D, const void* q, const void* k, const void* v, void* o, float scale,
                              void* stream);
/* Every option explicit: bf16 = 0 (fp16) / 1 (bfloat16); causal = 1 masks key j for
 * query i unless j <= i (key blocks above the diagonal are skipped).  The
 * reference's math has no mask (torch_attn.py:11-16); causal is an addition. */
int spork_attn_sm100_fwd_ex(int BH, int S, int D, const void* q, const void* k, const void* v, void* o, float scale,
                            int bf16, int causal, void* stream);

/* Reference-shaped FFI entry (tk_4090_fwd.hpp:7, called from
 * torch_attn.py:40-57): HOST fp32 (N, d) arrays, one head, scale 1/sqrt(d). */
void htod_f32_attn_sm100_fwd(int N, int d, const float* q, const float* k, const float* v, float* o);

/* Library/build information: "spork_b200 <version> sm_100a". */
const char* spork_b200_version(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* SPORK_B200_H */
