// Comparison column only, never part of libspork_b200.so: a CUTLASS GEMM for sm_100a (fp16 in, fp32
// accumulate and out, 256 x 256 x 64 tiles on CTA pairs, the library's own collective builders), built
// into a small shared object that the harness loads when it exists - the counterpart of the reference's
// matmul_cutlass / cutlass_enabled() (gemm/cutlass_gemm.h:5-6, gemm/cutlass_gemm.cu:42-131, an sm_90
// instantiation that does not compile for sm_100).  CUTLASS itself is not vendored here: the build step
// compiles this file only where a CUTLASS 4.x header tree is found (python -m spork_b200.build --cutlass).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "cutlass/cutlass.h"
#include "cute/tensor.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

using namespace cute;

using ElementA = cutlass::half_t;
using ElementB = cutlass::half_t;
using ElementC = float;
using ElementAcc = float;
using LayoutA = cutlass::layout::RowMajor;     // M x K, K contiguous
using LayoutB = cutlass::layout::ColumnMajor;  // K x N stored N x K, K contiguous
using LayoutC = cutlass::layout::RowMajor;
constexpr int AlignA = 8, AlignB = 8, AlignC = 4;

using TileShape = Shape<_256, _256, _64>;   // per CTA pair
using ClusterShape = Shape<_2, _1, _1>;

using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, TileShape, ClusterShape,
    cutlass::epilogue::collective::EpilogueTileAuto, ElementAcc, ElementAcc, ElementC, LayoutC, AlignC, ElementC, LayoutC,
    AlignC, cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;

using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, ElementA, LayoutA, AlignA, ElementB, LayoutB, AlignB, ElementAcc,
    TileShape, ClusterShape,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
    cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;

using GemmKernel =
    cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;

// 0 on success; 1 = shape not supported by this instantiation, 2 = workspace too small, 3 / 4 = CUTLASS
// initialisation / launch failed.  `workspace` is device memory the caller owns.
extern "C" __attribute__((visibility("default"))) size_t cutlass_sm100_workspace_bytes(uint32_t M, uint32_t N, uint32_t K)
{
    (void)M;
    (void)N;
    (void)K;
    return 64u << 20;  // ample for this instantiation (it needs a few KB of tile-scheduler state)
}

extern "C" __attribute__((visibility("default"))) int cutlass_sm100_f16f32(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, float* C,
                                    void* workspace, size_t workspace_bytes, cudaStream_t stream)
{
    using StrideA = typename Gemm::GemmKernel::StrideA;
    using StrideB = typename Gemm::GemmKernel::StrideB;
    using StrideC = typename Gemm::GemmKernel::StrideC;
    using StrideD = typename Gemm::GemmKernel::StrideD;
    StrideA sa = cutlass::make_cute_packed_stride(StrideA{}, cute::make_shape((int)M, (int)K, 1));
    StrideB sb = cutlass::make_cute_packed_stride(StrideB{}, cute::make_shape((int)N, (int)K, 1));
    StrideC sc = cutlass::make_cute_packed_stride(StrideC{}, cute::make_shape((int)M, (int)N, 1));
    StrideD sd = cutlass::make_cute_packed_stride(StrideD{}, cute::make_shape((int)M, (int)N, 1));
    typename Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                                  {(int)M, (int)N, (int)K, 1},
                                  {static_cast<const ElementA*>(A), sa, static_cast<const ElementB*>(B), sb},
                                  {{1.0f, 0.0f}, C, sc, C, sd}};
    Gemm gemm;
    if (gemm.can_implement(args) != cutlass::Status::kSuccess) {
        return 1;
    }
    if (Gemm::get_workspace_size(args) > workspace_bytes) {
        return 2;
    }
    if (gemm.initialize(args, workspace, stream) != cutlass::Status::kSuccess) {
        return 3;
    }
    return gemm.run(stream) == cutlass::Status::kSuccess ? 0 : 4;
}
