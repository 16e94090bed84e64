// COMPARISON INFRASTRUCTURE -- thin C driver around the reference's own sm_100 block-scaled GEMM kernels.
//
// This file contains no reference code: it includes the reference headers where they lie (the build passes
// -I<reference>/include -I<reference>/tools/util/include) and instantiates the kernel that the reference's
// CollectiveBuilder produces for the tile and cluster shape of its examples
// (examples/72_blackwell_narrow_precision_gemm/72a_blackwell_nvfp4_bf16_gemm.cu:120-151: MMA tile 256x256x256,
// cluster 2x4, automatic stage count and schedule; 72b_...:120-160 for the output with generated scale factors).
// It is the bar the hand-written kernel is measured against on the same GPU, with the same operands, by the same
// timing loop.  Built by baseline/Makefile into baseline/_ref/ (not tracked).  Nothing in the library loads it; only
// the reference arm of the benchmark does.
//
// REF_GPU_CONFIG: 0 = NVFP4 (e2m1, ue4m3 per 16) -> bf16;  1 = MXFP8 (e4m3, ue8m0 per 32) -> bf16;
//                 2 = NVFP4 -> e2m1 + generated ue4m3 scale factors per 16 (C is bf16, may be null).
#include <cstdint>
#include <cuda_runtime.h>

#include "cutlass/cutlass.h"
#include "cute/tensor.hpp"
#include "cutlass/tensor_ref.h"
#include "cutlass/epilogue/thread/linear_combination.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/detail/sm100_blockscaled_layout.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/gemm/kernel/tile_scheduler_params.h"
#include "cutlass/util/packed_stride.hpp"

#ifndef REF_GPU_CONFIG
#define REF_GPU_CONFIG 0
#endif
#ifndef REF_GPU_CLUSTER_N
#define REF_GPU_CLUSTER_N 4
#endif
#ifndef REF_GPU_MXFP8_TILE_K
#define REF_GPU_MXFP8_TILE_K 128
#endif

using namespace cute;

namespace {

#if REF_GPU_CONFIG == 1
using ElementA = cutlass::mx_float8_t<cutlass::float_e4m3_t>;
using ElementB = cutlass::mx_float8_t<cutlass::float_e4m3_t>;
constexpr int AlignmentAB = 16;
using MmaTileShape = Shape<_256, _256, Int<REF_GPU_MXFP8_TILE_K>>;
#else
using ElementA = cutlass::nv_float4_t<cutlass::float_e2m1_t>;
using ElementB = cutlass::nv_float4_t<cutlass::float_e2m1_t>;
constexpr int AlignmentAB = 32;
using MmaTileShape = Shape<_256, _256, _256>;
#endif
using ClusterShape = Shape<_2, Int<REF_GPU_CLUSTER_N>, _1>;
using ElementC = cutlass::bfloat16_t;
using LayoutRow = cutlass::layout::RowMajor;
using LayoutCol = cutlass::layout::ColumnMajor;
using ArchTag = cutlass::arch::Sm100;
using OpClass = cutlass::arch::OpClassBlockScaledTensorOp;
constexpr int AlignmentC = 8;

#if REF_GPU_CONFIG == 2
using ElementD = cutlass::float_e2m1_t;
using ElementSFD = cutlass::float_ue4m3_t;
constexpr int AlignmentD = 32;
using Fusion = cutlass::epilogue::fusion::LinCombBlockScaleFactor<16, ElementD, float, ElementSFD, LayoutRow, ElementC>;
using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    ArchTag, OpClass, MmaTileShape, ClusterShape, cutlass::epilogue::collective::EpilogueTileAuto, float, float,
    ElementC, LayoutRow, AlignmentC, ElementD, LayoutRow, AlignmentD,
    cutlass::epilogue::collective::EpilogueScheduleAuto, Fusion>::CollectiveOp;
#else
using ElementD = cutlass::bfloat16_t;
constexpr int AlignmentD = 8;
using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    ArchTag, OpClass, MmaTileShape, ClusterShape, cutlass::epilogue::collective::EpilogueTileAuto, float, float,
    ElementC, LayoutRow, AlignmentC, ElementD, LayoutRow, AlignmentD,
    cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;
#endif

using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    ArchTag, OpClass, ElementA, LayoutRow, AlignmentAB, ElementB, LayoutCol, AlignmentAB, float, MmaTileShape, ClusterShape,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
    cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;

using GemmKernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;
using StrideA = typename GemmKernel::StrideA;
using StrideB = typename GemmKernel::StrideB;
using StrideC = typename GemmKernel::StrideC;
using StrideD = typename GemmKernel::StrideD;
using SfConfig = typename CollectiveMainloop::Sm1xxBlkScaledConfig;

Gemm g_gemm;

typename Gemm::Arguments make_args(const void* A, const void* B, const void* SFA, const void* SFB, const void* C, void* D,
                                   void* SFD, const float* norm, int M, int N, int K, float alpha, float beta, int swizzle) {
  auto stride_A = cutlass::make_cute_packed_stride(StrideA{}, {M, K, 1});
  auto stride_B = cutlass::make_cute_packed_stride(StrideB{}, {N, K, 1});
  auto stride_C = cutlass::make_cute_packed_stride(StrideC{}, {M, N, 1});
  auto stride_D = cutlass::make_cute_packed_stride(StrideD{}, {M, N, 1});
  auto layout_SFA = SfConfig::tile_atom_to_shape_SFA(make_shape(M, N, K, 1));
  auto layout_SFB = SfConfig::tile_atom_to_shape_SFB(make_shape(M, N, K, 1));
  typename Gemm::Arguments args{
      cutlass::gemm::GemmUniversalMode::kGemm,
      {M, N, K, 1},
      {reinterpret_cast<const typename ElementA::DataType*>(A), stride_A,
       reinterpret_cast<const typename ElementB::DataType*>(B), stride_B,
       reinterpret_cast<const typename ElementA::ScaleFactorType*>(SFA), layout_SFA,
       reinterpret_cast<const typename ElementB::ScaleFactorType*>(SFB), layout_SFB},
      {{alpha, beta}, reinterpret_cast<const ElementC*>(C), stride_C, reinterpret_cast<ElementD*>(D), stride_D}};
#if REF_GPU_CONFIG == 2
  args.epilogue.thread.block_scale_factor_ptr = reinterpret_cast<ElementSFD*>(SFD);
  args.epilogue.thread.norm_constant_ptr = norm;
#else
  (void)SFD; (void)norm;
#endif
  args.scheduler.max_swizzle_size = swizzle;
  return args;
}

}  // namespace

extern "C" {

// Text description of the instantiated kernel (tile, cluster, stages).
const char* ref_gpu_describe() {
  static char buf[256];
  snprintf(buf, sizeof buf, "config %d mma_tile %dx%dx%d cluster 2x%dx1 stages %d smem %d", REF_GPU_CONFIG,
           int(size<0>(MmaTileShape{})), int(size<1>(MmaTileShape{})), int(size<2>(MmaTileShape{})), REF_GPU_CLUSTER_N,
           int(CollectiveMainloop::DispatchPolicy::Stages), int(GemmKernel::SharedStorageSize));
  return buf;
}

// Bytes of device workspace the kernel wants for this problem.
int64_t ref_gpu_workspace_size(int M, int N, int K) {
  auto args = make_args(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, M, N, K, 1.f, 0.f, 0);
  return int64_t(Gemm::get_workspace_size(args));
}

// can_implement + initialize (tensor maps, workspace).  Returns the cutlass::Status as an int (0 = success).
int ref_gpu_init(const void* A, const void* B, const void* SFA, const void* SFB, const void* C, void* D, void* SFD,
                 const float* norm, int M, int N, int K, float alpha, float beta, int swizzle, void* workspace,
                 cudaStream_t stream) {
  auto args = make_args(A, B, SFA, SFB, C, D, SFD, norm, M, N, K, alpha, beta, swizzle);
  cutlass::Status s = g_gemm.can_implement(args);
  if (s != cutlass::Status::kSuccess) return 1000 + int(s);
  s = g_gemm.initialize(args, workspace, stream);
  return int(s);
}

// One launch of the initialised kernel on `stream`.
int ref_gpu_launch(cudaStream_t stream) { return int(g_gemm.run(stream)); }

}  // extern "C"
