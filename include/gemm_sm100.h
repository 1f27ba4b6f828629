// C++ face of the sm_100a GEMM for the reference harness: the same by-value
// descriptor and launch-function shapes as gemm/gpu_tensor.h:9-21 (GPU_Tensors),
// gemm/gemm_sm90.h:14 (matmul_sm90) and gemm/gemm_sm80.h:5-6 (matmul_sm80,
// matmul_sm80_supports), with fp16 operands.  Header-only over the C ABI.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "spork_b200.h"

struct GPU_TensorsF16
{
    uint32_t M;
    uint32_t N;
    uint32_t K;
    __half const *a; /* pointer to GPU memory, M x K */
    __half const *b; /* pointer to GPU memory, N x K when b_col_major */
    float *c;        /* pointer to GPU memory, M x N */

    bool a_col_major;
    bool b_col_major;
    bool c_col_major;
};

// K split modes the sm_100a kernel offers; output_stationary and split_k_outer
// have the meaning of gemm_sm90_k_mode (gemm/gemm_sm90.h:5-12).
enum class gemm_sm100_k_mode
{
    output_stationary,
    split_k_outer,
    split_k_inner,  // the K ranges of a tile are neighbours in the schedule (gemm_sm90_k_mode::split_k_inner)
    stream_k,  // whole waves run tile by tile; the tiles of a last wave that is at most half full are cut
               // into aligned K ranges that run at the same time (the schedule of both
               // gemm_sm90_k_mode::stream_k_* flavours, which differ in code structure only)
    automatic, // output_stationary, split_k_outer with a split count chosen to fill the waves (few tiles, long
               // K), or stream_k (several waves, the last one less than half full); with variant 0 the tile
               // is the library's choice too
};

// The kernel takes the harness's hot operand layout: A row-major, B stored N x K (gemm/gemm_test.cu:365);
// K must be a multiple of 8.  C may be row-major or column-major: like matmul_sm90
// (gemm/gemm_sm90.cu:1349-1355) the other one is produced by exchanging the operands, C^T = B A^T.
inline bool matmul_sm100_supports(GPU_TensorsF16 t)
{
    return !t.a_col_major && t.b_col_major && spork_gemm_sm100_supports(t.M, t.N, t.K) != 0;
}

// Asynchronous on `stream`, like matmul_sm90.  Errors are printed, as the
// reference's launchers do, and also returned.
inline int matmul_sm100(GPU_TensorsF16 t, cudaStream_t stream, gemm_sm100_k_mode k_mode = gemm_sm100_k_mode::output_stationary,
                        int split_k = 1, int variant = 0)
{
    if (!matmul_sm100_supports(t)) {
        fprintf(stderr, "matmul_sm100: unsupported layout or K %% 8 != 0 (M=%u N=%u K=%u)\n", t.M, t.N, t.K);
        return SPORK_ERR_UNSUPPORTED_SHAPE;
    }
    if (t.c_col_major) {
        // a column-major M x N result is the row-major N x M result of the exchanged product
        const GPU_TensorsF16 swapped{t.N, t.M, t.K, t.b, t.a, t.c, false, true, false};
        t = swapped;
    }
    int rc;
    const bool is_split = (k_mode == gemm_sm100_k_mode::split_k_outer || k_mode == gemm_sm100_k_mode::split_k_inner) && split_k > 1;
    if (is_split || k_mode == gemm_sm100_k_mode::stream_k || k_mode == gemm_sm100_k_mode::automatic) {
        const int block_n = variant ? variant : (t.N <= 64 ? 64 : (t.N <= 128 ? 128 : 256));
        const int split = k_mode == gemm_sm100_k_mode::stream_k     ? -1
                          : k_mode == gemm_sm100_k_mode::automatic   ? 0
                          : k_mode == gemm_sm100_k_mode::split_k_inner ? -split_k
                                                                        : split_k;
        // automatic without a variant: the library picks the tile as well as the K mode
        const int cta_group = (k_mode == gemm_sm100_k_mode::automatic && variant == 0) ? 0 : 2;
        rc = spork_gemm_sm100_f16f32_ex(t.M, t.N, t.K, t.a, t.b, t.c, block_n, cta_group, split, 0, stream);
    } else {
        rc = spork_gemm_sm100_f16f32(t.M, t.N, t.K, t.a, t.b, t.c, variant, stream);
    }
    if (rc != 0) {
        fprintf(stderr, "matmul_sm100: error %d\n", rc);
    }
    return rc;
}

// L independent products in one launch; `t` describes one of them and the L matrices of each operand
// follow one another in memory: the batch dimension of the reference's generated entry points
// (xgemm_Sm90.py:45-48, called with L = 1 at gemm/gemm_test.cu:310-362).
inline int matmul_sm100_batched(uint32_t L, GPU_TensorsF16 t, cudaStream_t stream, int split_k = 1, int variant = 0)
{
    if (!matmul_sm100_supports(t)) {
        fprintf(stderr, "matmul_sm100_batched: unsupported layout or K %% 8 != 0 (M=%u N=%u K=%u)\n", t.M, t.N, t.K);
        return SPORK_ERR_UNSUPPORTED_SHAPE;
    }
    const int rc = spork_gemm_sm100_f16f32_batched(L, t.M, t.N, t.K, t.a, t.b, t.c, variant, split_k, stream);
    if (rc != 0) {
        fprintf(stderr, "matmul_sm100_batched: error %d\n", rc);
    }
    return rc;
}

// Drop-in for the reference's own descriptor type: `Tensors` is any by-value struct with the fields of
// GPU_Tensors (gemm/gpu_tensor.h:9-21: M, N, K, float const* a, b, float* c, a_col_major, b_col_major,
// c_col_major), so `matmul_sm100_tf32(t, stream)` can stand where `matmul_sm90(t, mode, stream)`
// (gemm/gemm_sm90.h:14) or `matmul_sm80(t, stream)` (gemm/gemm_sm80.h:5) stands.  Operands are read as
// tf32, as those kernels read them.  Like matmul_sm90 it takes A row-major and B stored N x K
// (gemm/gemm_sm90.cu:1269-1270); a column-major C is produced by exchanging the operands.
template <class Tensors>
inline bool matmul_sm100_tf32_supports(Tensors t)
{
    return !t.a_col_major && t.b_col_major && t.K % 4 == 0;
}

template <class Tensors>
inline int matmul_sm100_tf32(Tensors t, cudaStream_t stream, int split_k = 1)
{
    if (!matmul_sm100_tf32_supports(t)) {
        fprintf(stderr, "matmul_sm100_tf32: unsupported layout or K %% 4 != 0 (M=%u N=%u K=%u)\n", t.M, t.N, t.K);
        return SPORK_ERR_UNSUPPORTED_SHAPE;
    }
    // C^T = B A^T: a column-major M x N result is the row-major N x M result of the exchanged product
    const int rc = t.c_col_major ? spork_gemm_sm100_tf32f32(t.N, t.M, t.K, t.b, t.a, t.c, 0, split_k, stream)
                                 : spork_gemm_sm100_tf32f32(t.M, t.N, t.K, t.a, t.b, t.c, 0, split_k, stream);
    if (rc != 0) {
        fprintf(stderr, "matmul_sm100_tf32: error %d\n", rc);
    }
    return rc;
}

inline int matmul_baseline_f16(GPU_TensorsF16 t, cudaStream_t stream)
{
    return spork_gemm_baseline_f16f32(t.M, t.N, t.K, t.a, t.b, t.c, stream);
}
