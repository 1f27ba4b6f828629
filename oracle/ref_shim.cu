// C-ABI shim around the reference's own launch functions, so that Python can
// call them with ctypes.  Test infrastructure only.  Compiled together with the
// reference's unmodified gemm/gemm_baseline.cu and gemm/gemm_sm80.cu (found
// through -I <reference>/gemm; nothing is copied) into oracle/_ref/.
//
//   matmul_baseline  gemm/gemm_baseline.h:5   fp32 FFMA, the reference's oracle
//   matmul_sm80      gemm/gemm_sm80.h:5-6     mma.sync TF32, Ampere-generation
#include "gemm_baseline.h"
#include "gemm_sm80.h"

#define REF_API extern "C" __attribute__((visibility("default")))

static GPU_Tensors make(uint32_t M, uint32_t N, uint32_t K, const float* a, const float* b, float* c, int a_col,
                        int b_col, int c_col)
{
    GPU_Tensors t{};
    t.M = M;
    t.N = N;
    t.K = K;
    t.a = a;
    t.b = b;
    t.c = c;
    t.a_col_major = a_col != 0;
    t.b_col_major = b_col != 0;
    t.c_col_major = c_col != 0;
    return t;
}

REF_API int spork_ref_matmul_baseline(uint32_t M, uint32_t N, uint32_t K, const float* a, const float* b, float* c,
                                      int a_col, int b_col, int c_col, void* stream)
{
    matmul_baseline(make(M, N, K, a, b, c, a_col, b_col, c_col), static_cast<cudaStream_t>(stream));
    return (int)cudaGetLastError();
}

REF_API int spork_ref_matmul_sm80_supports(uint32_t M, uint32_t N, uint32_t K)
{
    return matmul_sm80_supports(make(M, N, K, nullptr, nullptr, nullptr, 0, 1, 0)) ? 1 : 0;
}

REF_API int spork_ref_matmul_sm80(uint32_t M, uint32_t N, uint32_t K, const float* a, const float* b, float* c,
                                  int a_col, int b_col, int c_col, void* stream)
{
    matmul_sm80(make(M, N, K, a, b, c, a_col, b_col, c_col), static_cast<cudaStream_t>(stream));
    return (int)cudaGetLastError();
}
