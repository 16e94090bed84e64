// Block-scaled quantiser: bf16 (rows x K, row-major) -> NVFP4 or MXFP8 values plus scale factors
// in the interleaved layout the GEMM reads (512-byte atoms of 128 rows x 4 K-blocks).
//
// The arithmetic is the reference's block-scale computation
// (tools/util/include/cutlass/util/reference/host/gett.hpp:436-478): per row and K-block of V elements
//   amax -> SF = cvt(amax * (st * (1 / fp_max))) -> q = cvt(x * min(st * (1 / float(SF)), FLT_MAX)),
// every product separately rounded.  NVFP4: V = 16, SF ue4m3, q e2m1 (fp_max 6);  MXFP8: V = 32,
// SF ue8m0 (the conversion rounds up), q e4m3 (fp_max 448).
//
// HBM-bound.  One CTA owns a tile of 128 rows x 256 elements: a warp reads one row of the tile per
// step as 32 x 16 bytes (fully coalesced), the lanes that share a K-block combine their maxima with
// shuffles, and every lane stores its own 8 quantised values (4 or 8 bytes, coalesced).  The tile's
// scale factors are collected in shared memory in atom order and leave as whole 512-byte atoms.
// (Tiles of 128 x 128, which fill the last wave of an 8192 x 8192 operand better, were measured slower at
// every size: the per-CTA set-up and the atom write-out weigh more than the emptier last wave.)
// Maximum and minimum propagate NaN as the reference's do (maximum_with_nan_propogation, gett.hpp:390): one NaN
// in a block turns its scale factor and all of its values into NaN codes (e2m1 has none: the largest value).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cfloat>
#include <cstdint>

#include "ptx.cuh"

namespace bsg {

struct QuantParams {
  const uint16_t* X;      // bf16 bits
  uint8_t* Q;
  uint8_t* SF;
  const float* norm_ptr;  // device scalar st, or null for 1.0
  int64_t ldx;            // elements between rows of X
  int32_t rows, K;
  int32_t k_atoms;        // ceil(K / V / 4)
};

constexpr int kQuantTileRows = 128;
constexpr int kQuantTileK = 256;
constexpr int kQuantThreads = 256;

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
// max of two packed bf16 pairs, element-wise; a NaN operand gives NaN.
__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_absmax(uint32_t a, uint32_t b) { return bf16x2_max(a & 0x7FFF7FFFu, b & 0x7FFF7FFFu); }

template <int KIND>
__global__ void __launch_bounds__(kQuantThreads, 4) bsg_quant_kernel(const QuantParams p) {
  constexpr int V = KIND == 0 ? 16 : 32;
  constexpr int kLanesPerBlock = V / 8;                     // lanes that share one K-block
  constexpr int kBlocksPerTile = kQuantTileK / V;           // K-blocks of one row of the tile: 16 or 8
  constexpr int kAtomsPerTile = kBlocksPerTile / 4;         // 4 or 2
  __shared__ __align__(16) uint8_t s_sf[kAtomsPerTile * 512];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.y * kQuantTileRows;
  const int k0 = blockIdx.x * kQuantTileK;
  for (int i = threadIdx.x; i < kAtomsPerTile * 512 / 4; i += kQuantThreads) reinterpret_cast<uint32_t*>(s_sf)[i] = 0u;
  __syncthreads();

  const float st = p.norm_ptr ? *p.norm_ptr : 1.0f;
  const float st_scaled = __fmul_rn(st, __fdiv_rn(1.0f, KIND == 0 ? 6.0f : 448.0f));
  const int k = k0 + lane * 8;
  const bool k_ok = k < p.K;
  const int blk = lane / kLanesPerBlock;                    // K-block of this lane inside the tile row

  // A warp owns rows warp + 8 u + 32 g of the tile (u < 4, g < 4).  The four loads of group g + 1 are issued
  // before group g is processed, so that every warp always has loads in flight (the kernel is bound by
  // memory latency x bytes in flight, not by arithmetic).
  constexpr int kUnroll = 4, kGroups = kQuantTileRows / (8 * kUnroll);
  auto load_group = [&](uint4 (&raw)[kUnroll], int g) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int row = row0 + warp + 8 * u + 32 * g;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (k_ok && row < p.rows) raw[u] = *reinterpret_cast<const uint4*>(p.X + int64_t(row) * p.ldx + k);
    }
  };
  uint4 raw[kUnroll], nxt[kUnroll];
  load_group(raw, 0);
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    if (g + 1 < kGroups) load_group(nxt, g + 1);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int rt = warp + 8 * u + 32 * g, row = row0 + rt;
      float x[8];
      x[0] = bf16_bits_to_f32(raw[u].x & 0xFFFFu); x[1] = bf16_bits_to_f32(raw[u].x >> 16);
      x[2] = bf16_bits_to_f32(raw[u].y & 0xFFFFu); x[3] = bf16_bits_to_f32(raw[u].y >> 16);
      x[4] = bf16_bits_to_f32(raw[u].z & 0xFFFFu); x[5] = bf16_bits_to_f32(raw[u].z >> 16);
      x[6] = bf16_bits_to_f32(raw[u].w & 0xFFFFu); x[7] = bf16_bits_to_f32(raw[u].w >> 16);
      // |x| maximum of the lane's 8 values on the packed bf16 pairs (exact: max and abs do not round)
      const uint32_t m01 = bf16x2_absmax(raw[u].x, raw[u].y), m23 = bf16x2_absmax(raw[u].z, raw[u].w);
      const uint32_t m = bf16x2_max(m01, m23);
      float amax = ptx::fmax_nan(bf16_bits_to_f32(m & 0xFFFFu), bf16_bits_to_f32(m >> 16));
      amax = ptx::fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      if constexpr (kLanesPerBlock == 4) amax = ptx::fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const float pv = __fmul_rn(amax, st_scaled);
      uint32_t sf_code;
      float sf_val;
      if constexpr (KIND == 0) {
        sf_code = ptx::cvt_ue4m3(pv);
        sf_val = ptx::cvt_e4m3_to_f32(sf_code);
      } else {
        sf_code = ptx::cvt_ue8m0_rp(pv);
        sf_val = ptx::ue8m0_to_f32(sf_code);
      }
      float sc = __fmul_rn(st, __frcp_rn(sf_val));      // correctly rounded reciprocal == 1.0f / sf_val
      sc = ptx::fmin_nan(sc, FLT_MAX);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(x[j], sc);
      if (k_ok && row < p.rows) {
        if constexpr (KIND == 0) {
          *reinterpret_cast<uint32_t*>(p.Q + int64_t(row) * (p.K / 2) + k / 2) = ptx::cvt_e2m1x8(x);
        } else {
          uint2 q;
          q.x = ptx::cvt_e4m3x4(x[0], x[1], x[2], x[3]);
          q.y = ptx::cvt_e4m3x4(x[4], x[5], x[6], x[7]);
          *reinterpret_cast<uint2*>(p.Q + int64_t(row) * p.K + k) = q;
        }
        if ((lane % kLanesPerBlock) == 0)
          s_sf[(blk >> 2) * 512 + 16 * (rt & 31) + 4 * (rt >> 5) + (blk & 3)] = uint8_t(sf_code);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) raw[u] = nxt[u];
  }
  __syncthreads();
  // Whole atoms leave in one piece: atom (row0 / 128, k0 / (4 V) + a), 512 bytes each, consecutive in memory.
  const int atom0 = k0 / (4 * V);
  const int n_atoms = min(kAtomsPerTile, p.k_atoms - atom0);
  uint8_t* dst = p.SF + (int64_t(blockIdx.y) * p.k_atoms + atom0) * 512;
  for (int i = threadIdx.x; i < n_atoms * 32; i += kQuantThreads)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(s_sf)[i];
}

}  // namespace bsg
