// TEST INFRASTRUCTURE -- thin C driver around the reference's own host GEMM.
//
// This file contains no reference code: it includes the reference headers where
// they lie (the build passes -I<reference>/include -I<reference>/tools/util/include)
// and instantiates cutlass::reference::host::Gemm3x
// (tools/util/include/cutlass/util/reference/host/gett.hpp:837) with the block-scaled
// parameter structs (gett.hpp:132,279), the reference's numeric types
// (include/cutlass/float8.h, float_subbyte.h) and its scale-factor layouts
// (include/cutlass/detail/sm100_blockscaled_layout.hpp:62,192).
// Built by oracle/Makefile into oracle/_ref/libbsg_ref.so.  Only tests, the smoke
// check and the CPU-baseline leg of the benchmark may load it.
#include <cstdint>
#include <cstring>

#include "cutlass/cutlass.h"
#include "cutlass/numeric_types.h"
#include "cutlass/detail/sm100_blockscaled_layout.hpp"
#include "cutlass/util/reference/host/gett.hpp"
#include "cute/tensor.hpp"

using namespace cute;

namespace {

template <int Vec>
using SfCfg = cutlass::detail::Sm1xxBlockScaledConfig<Vec>;
template <int Vec>
using SfOutCfg = cutlass::detail::Sm1xxBlockScaledOutputConfig<Vec>;
template <int Vec>
using SfOutCfgColMajor = cutlass::detail::Sm1xxBlockScaledOutputConfig<Vec, cute::UMMA::Major::MN>;

template <class ElemAB, class ElemSF, int Vec, class ElemD, bool GenSfd, int SfdVec = 16, class ElemSFD = cutlass::float_ue4m3_t,
          class ElemB = ElemAB, bool ColMajorD = false>
void run_gemm(int M, int N, int K, const void* A, const void* B, const void* SFA, const void* SFB,
              const cutlass::bfloat16_t* C, float alpha, float beta, void* D, void* SFD, float st) {
  auto layout_A = make_layout(make_shape(M, K, 1), make_stride(int64_t(K), _1{}, int64_t(M) * K));
  auto layout_B = make_layout(make_shape(N, K, 1), make_stride(int64_t(K), _1{}, int64_t(N) * K));
  auto layout_C = make_layout(make_shape(M, N, 1), make_stride(int64_t(N), _1{}, int64_t(M) * N));
  auto layout_SFA = SfCfg<Vec>::tile_atom_to_shape_SFA(make_shape(M, N, K, 1));
  auto layout_SFB = SfCfg<Vec>::tile_atom_to_shape_SFB(make_shape(M, N, K, 1));

  Tensor tA = make_tensor(recast_ptr<ElemAB>(const_cast<void*>(A)), layout_A);
  Tensor tB = make_tensor(recast_ptr<ElemB>(const_cast<void*>(B)), layout_B);
  Tensor tSFA = make_tensor(reinterpret_cast<ElemSF*>(const_cast<void*>(SFA)), layout_SFA);
  Tensor tSFB = make_tensor(reinterpret_cast<ElemSF*>(const_cast<void*>(SFB)), layout_SFB);
  cutlass::reference::host::GettBlockScalingMainloopParams<float, decltype(tA), decltype(tSFA), decltype(tB), decltype(tSFB)>
      mainloop{tA, tSFA, tB, tSFB};

  Tensor tC = make_tensor(const_cast<cutlass::bfloat16_t*>(C), layout_C);
  if constexpr (GenSfd && ColMajorD) {
    // D stored column-major (M contiguous), scale factors per SfdVec consecutive ROWS of a column, in the
    // reference's M-major scale-factor layout (the branch of gett.hpp:392-430)
    auto layout_D = make_layout(make_shape(M, N, 1), make_stride(_1{}, int64_t(M), int64_t(M) * N));
    Tensor tD = make_tensor(recast_ptr<ElemD>(D), layout_D);
    auto layout_SFD = SfOutCfgColMajor<SfdVec>::tile_atom_to_shape_SFD(make_shape(M, N, K, 1));
    Tensor tSFD = make_tensor(reinterpret_cast<ElemSFD*>(SFD), layout_SFD);
    cutlass::reference::host::GettBlockScalingEpilogueParams<float, float, float, decltype(tC), decltype(tD), decltype(tSFD),
                                                             cute::Int<SfdVec>, cutlass::reference::host::SfStrategy::SfDGen>
        epi{alpha, beta, tC, tD, tSFD, st};
    cutlass::reference::host::Gemm3x(mainloop, epi);
    return;
  }
  Tensor tD = make_tensor(recast_ptr<ElemD>(D), layout_C);
  if constexpr (GenSfd) {
    auto layout_SFD = SfOutCfg<SfdVec>::tile_atom_to_shape_SFD(make_shape(M, N, K, 1));
    Tensor tSFD = make_tensor(reinterpret_cast<ElemSFD*>(SFD), layout_SFD);
    cutlass::reference::host::GettBlockScalingEpilogueParams<float, float, float, decltype(tC), decltype(tD), decltype(tSFD),
                                                             cute::Int<SfdVec>, cutlass::reference::host::SfStrategy::SfDGen>
        epi{alpha, beta, tC, tD, tSFD, st};
    cutlass::reference::host::Gemm3x(mainloop, epi);
  } else {
    cutlass::reference::host::GettBlockScalingEpilogueParams<float, float, float, decltype(tC), decltype(tD)> epi{alpha, beta, tC, tD};
    cutlass::reference::host::Gemm3x(mainloop, epi);
  }
}

// The general host epilogue of the reference (GettEpilogueParams, gett.hpp:173-262): bias vector, beta * C and an
// activation functor of include/cutlass/epilogue/thread/activation.h; D in fp32.
template <class ElemAB, class ElemSF, int Vec, class Act, bool PerCol>
void run_gemm_epi(int M, int N, int K, const void* A, const void* B, const void* SFA, const void* SFB,
                  const cutlass::bfloat16_t* C, float alpha, float beta, const float* bias, float* D) {
  auto layout_A = make_layout(make_shape(M, K, 1), make_stride(int64_t(K), _1{}, int64_t(M) * K));
  auto layout_B = make_layout(make_shape(N, K, 1), make_stride(int64_t(K), _1{}, int64_t(N) * K));
  auto layout_C = make_layout(make_shape(M, N, 1), make_stride(int64_t(N), _1{}, int64_t(M) * N));
  auto layout_SFA = SfCfg<Vec>::tile_atom_to_shape_SFA(make_shape(M, N, K, 1));
  auto layout_SFB = SfCfg<Vec>::tile_atom_to_shape_SFB(make_shape(M, N, K, 1));
  Tensor tA = make_tensor(recast_ptr<ElemAB>(const_cast<void*>(A)), layout_A);
  Tensor tB = make_tensor(recast_ptr<ElemAB>(const_cast<void*>(B)), layout_B);
  Tensor tSFA = make_tensor(reinterpret_cast<ElemSF*>(const_cast<void*>(SFA)), layout_SFA);
  Tensor tSFB = make_tensor(reinterpret_cast<ElemSF*>(const_cast<void*>(SFB)), layout_SFB);
  cutlass::reference::host::GettBlockScalingMainloopParams<float, decltype(tA), decltype(tSFA), decltype(tB), decltype(tSFB)>
      mainloop{tA, tSFA, tB, tSFB};
  Tensor tC = make_tensor(const_cast<cutlass::bfloat16_t*>(C), layout_C);
  Tensor tD = make_tensor(D, layout_C);
  Tensor tBias = make_tensor(const_cast<float*>(bias), make_layout(make_shape(PerCol ? N : M, 1, 1)));
  using Unused = decltype(make_tensor(cute::recast_ptr<float>(nullptr), typename decltype(tD)::layout_type{}));
  using Epi = cutlass::reference::host::GettEpilogueParams<float, float, float, float, decltype(tC), decltype(tD), decltype(tBias),
                                                           Unused, Unused, Unused, Act, decltype(tD), cute::Int<0>,
                                                           cutlass::plus<float>, PerCol>;
  Epi epi;
  epi.alpha = alpha;
  epi.beta = beta;
  epi.C = tC;
  epi.D = tD;
  epi.Bias = tBias;
  cutlass::reference::host::Gemm3x(mainloop, epi);
}

template <class ElemAB, class ElemSF, int Vec>
int dispatch_epi(int M, int N, int K, const void* A, const void* B, const void* SFA, const void* SFB,
                 const cutlass::bfloat16_t* C, float alpha, float beta, const float* bias, int bias_mode, int act, float* D) {
  using namespace cutlass::epilogue::thread;
  const bool per_col = bias_mode != 2;
  const float* b = bias_mode == 0 ? nullptr : bias;
#define BSG_EPI(ACT) (per_col ? run_gemm_epi<ElemAB, ElemSF, Vec, ACT<float>, true>(M, N, K, A, B, SFA, SFB, C, alpha, beta, b, D) \
                              : run_gemm_epi<ElemAB, ElemSF, Vec, ACT<float>, false>(M, N, K, A, B, SFA, SFB, C, alpha, beta, b, D))
  switch (act) {
    case 0: BSG_EPI(Identity); return 0;
    case 1: BSG_EPI(ReLu); return 0;
    case 2: BSG_EPI(GELU); return 0;
    case 3: BSG_EPI(SiLu); return 0;
    default: return 1;
  }
#undef BSG_EPI
}

}  // namespace

extern "C" {

// fmt: 0 e2m1 (4-bit code), 1 e4m3, 2 ue4m3, 3 ue8m0, 4 e5m2
float bsg_ref_decode(int fmt, uint32_t code) {
  switch (fmt) {
    case 4: return float(cutlass::float_e5m2_t::bitcast(uint8_t(code)));
    case 0: return float(cutlass::float_e2m1_t::bitcast(uint8_t(code & 0xF)));
    case 1: return float(cutlass::float_e4m3_t::bitcast(uint8_t(code)));
    case 2: return float(cutlass::float_ue4m3_t::bitcast(uint8_t(code)));
    default: return float(cutlass::float_ue8m0_t::bitcast(uint8_t(code)));
  }
}

uint32_t bsg_ref_encode(int fmt, float x) {
  switch (fmt) {
    case 4: return cutlass::float_e5m2_t(x).raw();
    case 0: return cutlass::float_e2m1_t(x).raw() & 0xF;
    case 1: return cutlass::float_e4m3_t(x).raw();
    case 2: return cutlass::float_ue4m3_t(x).raw();
    default: return cutlass::float_ue8m0_t(x).raw();
  }
}

// Element offset of the scale factor of (row, k) in the SFA layout of an (rows x K) operand.
int64_t bsg_ref_sf_offset(int vec, int rows, int K, int row, int k) {
  if (vec == 16) {
    auto l = SfCfg<16>::tile_atom_to_shape_SFA(make_shape(rows, 1, K, 1));
    return int64_t(l(row, k, 0));
  }
  auto l = SfCfg<32>::tile_atom_to_shape_SFA(make_shape(rows, 1, K, 1));
  return int64_t(l(row, k, 0));
}

int64_t bsg_ref_sf_size(int vec, int rows, int K) {
  if (vec == 16) return int64_t(size(filter_zeros(SfCfg<16>::tile_atom_to_shape_SFA(make_shape(rows, 1, K, 1)))));
  return int64_t(size(filter_zeros(SfCfg<32>::tile_atom_to_shape_SFA(make_shape(rows, 1, K, 1)))));
}

// kind 0 NVFP4 / 1 MXFP8 / 2 MXFP4 / 3 mixed (A e4m3, B e2m1; out_mode 0 and 1 only for 2 and 3).  out_mode 0: D fp32, 1: D bf16, 2: D e2m1 + SFD ue4m3 per 16 (NVFP4 re-quantisation with norm
// constant st), 3: D e4m3 + SFD ue8m0 per 32 (MXFP8 re-quantisation); 4 / 5 (kind 0 only): as 2 / 3 with D stored
// column-major (M contiguous) and the scale factors per 16 / 32 consecutive rows of a column.
// C is bf16 (may be null when beta == 0).  Returns 0 on success.
int bsg_ref_gemm(int kind, int out_mode, int M, int N, int K, const void* A, const void* B, const void* SFA, const void* SFB,
                 const void* C, float alpha, float beta, void* D, void* SFD, float st) {
  auto Cb = static_cast<const cutlass::bfloat16_t*>(C);
  if (kind == 0) {
    using E = cutlass::float_e2m1_t;
    using S = cutlass::float_ue4m3_t;
    if (out_mode == 0) run_gemm<E, S, 16, float, false>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, nullptr, 0.f);
    else if (out_mode == 1) run_gemm<E, S, 16, cutlass::bfloat16_t, false>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, nullptr, 0.f);
    else if (out_mode == 2) run_gemm<E, S, 16, cutlass::float_e2m1_t, true>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, SFD, st);
    else if (out_mode == 3) run_gemm<E, S, 16, cutlass::float_e4m3_t, true, 32, cutlass::float_ue8m0_t>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, SFD, st);
    else if (out_mode == 4) run_gemm<E, S, 16, cutlass::float_e2m1_t, true, 16, cutlass::float_ue4m3_t, E, true>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, SFD, st);
    else if (out_mode == 5) run_gemm<E, S, 16, cutlass::float_e4m3_t, true, 32, cutlass::float_ue8m0_t, E, true>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, SFD, st);
    else return 1;
  } else if (kind == 1) {
    using E = cutlass::float_e4m3_t;
    using S = cutlass::float_ue8m0_t;
    if (out_mode == 0) run_gemm<E, S, 32, float, false>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, nullptr, 0.f);
    else if (out_mode == 1) run_gemm<E, S, 32, cutlass::bfloat16_t, false>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, nullptr, 0.f);
    else if (out_mode == 2) run_gemm<E, S, 32, cutlass::float_e2m1_t, true>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, SFD, st);
    else if (out_mode == 3) run_gemm<E, S, 32, cutlass::float_e4m3_t, true, 32, cutlass::float_ue8m0_t>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, SFD, st);
    else return 1;
  } else if (kind == 2 || kind == 3) {
    // MXFP4 (e2m1 x e2m1) and the mixed form of the reference's example 72c (A e4m3, B e2m1); ue8m0 scale per 32.
    using S = cutlass::float_ue8m0_t;
    using F4 = cutlass::float_e2m1_t;
    using F8 = cutlass::float_e4m3_t;
    if (kind == 2) {
      if (out_mode == 0) run_gemm<F4, S, 32, float, false>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, nullptr, 0.f);
      else if (out_mode == 1) run_gemm<F4, S, 32, cutlass::bfloat16_t, false>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, nullptr, 0.f);
      else return 1;
    } else {
      if (out_mode == 0) run_gemm<F8, S, 32, float, false, 16, cutlass::float_ue4m3_t, F4>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, nullptr, 0.f);
      else if (out_mode == 1) run_gemm<F8, S, 32, cutlass::bfloat16_t, false, 16, cutlass::float_ue4m3_t, F4>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, D, nullptr, 0.f);
      else return 1;
    }
  } else {
    return 1;
  }
  return 0;
}

// fp32 D = act(alpha * acc + bias + beta * C).  bias_mode 0 none, 1 per column, 2 per row; act 0 identity, 1 ReLU, 2 GELU, 3 SiLU.
int bsg_ref_gemm_epi(int kind, int M, int N, int K, const void* A, const void* B, const void* SFA, const void* SFB, const void* C,
                     float alpha, float beta, const float* bias, int bias_mode, int act, float* D) {
  auto Cb = static_cast<const cutlass::bfloat16_t*>(C);
  if (kind == 0) return dispatch_epi<cutlass::float_e2m1_t, cutlass::float_ue4m3_t, 16>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, bias, bias_mode, act, D);
  if (kind == 1) return dispatch_epi<cutlass::float_e4m3_t, cutlass::float_ue8m0_t, 32>(M, N, K, A, B, SFA, SFB, Cb, alpha, beta, bias, bias_mode, act, D);
  return 1;
}

}  // extern "C"
