// Block-scaled quantiser: bf16 (rows x K, row-major) -> NVFP4 or MXFP8 values plus scale factors
// in the interleaved layout the GEMM reads (512-byte atoms of 128 rows x 4 K-blocks).
//
// The arithmetic is the reference's block-scale computation
// (tools/util/include/cutlass/util/reference/host/gett.hpp:436-478): per row and K-block of V elements
//   amax -> SF = cvt(amax * (st * (1 / fp_max))) -> q = cvt(x * min(st * (1 / float(SF)), FLT_MAX)),
// every product separately rounded.  NVFP4: V = 16, SF ue4m3, q e2m1 (fp_max 6);  MXFP8: V = 32,
// SF ue8m0 (the conversion rounds up), q e4m3 (fp_max 448).
//
// HBM-bound.  One CTA owns a tile of 128 rows x 256 elements.  A lane owns one whole K-block of a row (16 or 32
// values: 32 or 64 bytes, fetched with 256-bit loads where the row addresses allow), so the block maximum needs no
// shuffle and the scale arithmetic is done once per block; a warp covers two (NVFP4) or four (MXFP8) rows per step.
// The tile's scale factors are collected in shared memory in atom order and leave as whole 512-byte atoms.
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
// magnitude of the result = max(|a|, |b|) per half (the sign is the xor of the operands' signs: masked off at the end)
__device__ __forceinline__ uint32_t bf16x2_maxabs(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ void ld_global_32B(uint32_t (&v)[8], const void* p, bool wide) {
  if (wide) {
    asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(p));
  } else {
    const uint4 lo = reinterpret_cast<const uint4*>(p)[0], hi = reinterpret_cast<const uint4*>(p)[1];
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
  }
}

template <int KIND>
__global__ void __launch_bounds__(kQuantThreads, 4) bsg_quant_kernel(const QuantParams p) {
  constexpr int V = KIND == 0 ? 16 : 32;                    // values per lane = one K-block
  constexpr int kWords = V / 2;                             // 32-bit words of bf16 pairs per lane and row
  constexpr int kLanesPerRow = kQuantTileK / V;             // 16 or 8
  constexpr int kRowsPerStep = 32 / kLanesPerRow;           // rows a warp covers with one step: 2 or 4
  constexpr int kSteps = kQuantTileRows / 8 / kRowsPerStep; // steps per warp: 8 or 4
  constexpr int kUnroll = 16 / kWords;                      // steps per group (16 words of loads in flight per group): 2 or 1
  constexpr int kGroups = kSteps / kUnroll;                 // 4
  constexpr int kAtomsPerTile = kLanesPerRow / 4;           // 4 or 2
  __shared__ __align__(16) uint8_t s_sf[kAtomsPerTile * 512];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.y * kQuantTileRows;
  const int k0 = blockIdx.x * kQuantTileK;
  for (int i = threadIdx.x; i < kAtomsPerTile * 512 / 4; i += kQuantThreads) reinterpret_cast<uint32_t*>(s_sf)[i] = 0u;
  __syncthreads();
  // Programmatic dependent launch (no-ops otherwise): X may come from the kernel before this one on the stream, which
  // must be complete before the first read; the kernel after this one may begin its own set-up right away.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  const float st = p.norm_ptr ? *p.norm_ptr : 1.0f;
  const float st_scaled = __fmul_rn(st, __fdiv_rn(1.0f, KIND == 0 ? 6.0f : 448.0f));
  const int blk = lane % kLanesPerRow;                      // K-block of this lane inside the tile row
  const int sub = lane / kLanesPerRow;                      // row of the step
  const int k = k0 + blk * V;
  const bool k_ok = k < p.K;
  // 256-bit accesses need 32-byte aligned rows
  const bool wide_in = ((reinterpret_cast<uintptr_t>(p.X) & 31u) == 0) && (p.ldx % 16 == 0);
  const bool wide_out = (reinterpret_cast<uintptr_t>(p.Q) & 31u) == 0;

  // Step s of a warp covers tile rows (s * 8 + warp) * kRowsPerStep + sub.  The loads of group g + 1 are issued before
  // group g is processed, so that every warp always has loads in flight.
  auto tile_row = [&](int g, int u) { return ((g * kUnroll + u) * 8 + warp) * kRowsPerStep + sub; };
  auto load_group = [&](uint32_t (&raw)[kUnroll][kWords], int g) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int row = row0 + tile_row(g, u);
#pragma unroll
      for (int j = 0; j < kWords; ++j) raw[u][j] = 0u;
      if (k_ok && row < p.rows) {
        const uint16_t* src = p.X + int64_t(row) * p.ldx + k;
#pragma unroll
        for (int h = 0; h < kWords / 8; ++h) ld_global_32B(*reinterpret_cast<uint32_t(*)[8]>(&raw[u][h * 8]), src + h * 16, wide_in);
      }
    }
  };
  uint32_t raw[kUnroll][kWords], nxt[kUnroll][kWords];
  load_group(raw, 0);
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    if (g + 1 < kGroups) load_group(nxt, g + 1);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int rt = tile_row(g, u), row = row0 + rt;
      // |x| maximum of the block on the packed bf16 pairs (exact: max and abs do not round)
      uint32_t m[kWords];
#pragma unroll
      for (int j = 0; j < kWords; ++j) m[j] = raw[u][j];
#pragma unroll
      for (int w = kWords / 2; w >= 1; w >>= 1) {
#pragma unroll
        for (int j = 0; j < w; ++j) m[j] = bf16x2_maxabs(m[j], m[j + w]);
      }
      const uint32_t mm = m[0] & 0x7FFF7FFFu;
      const float amax = ptx::fmax_nan(bf16_bits_to_f32(mm & 0xFFFFu), bf16_bits_to_f32(mm >> 16));
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
      uint32_t q[kWords / 4];                           // NVFP4: 8 values per word; MXFP8: 4 values per word -> kWords / 2 words
      uint32_t q8[kWords / 2];
#pragma unroll
      for (int c = 0; c < kWords / 4; ++c) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          x[2 * j] = __fmul_rn(bf16_bits_to_f32(raw[u][c * 4 + j] & 0xFFFFu), sc);
          x[2 * j + 1] = __fmul_rn(bf16_bits_to_f32(raw[u][c * 4 + j] >> 16), sc);
        }
        if constexpr (KIND == 0) {
          q[c] = ptx::cvt_e2m1x8(x);
        } else {
          q8[2 * c] = ptx::cvt_e4m3x4(x[0], x[1], x[2], x[3]);
          q8[2 * c + 1] = ptx::cvt_e4m3x4(x[4], x[5], x[6], x[7]);
        }
      }
      if (k_ok && row < p.rows) {
        if constexpr (KIND == 0) {
          *reinterpret_cast<uint2*>(p.Q + int64_t(row) * (p.K / 2) + k / 2) = make_uint2(q[0], q[1]);
        } else {
          uint8_t* dst = p.Q + int64_t(row) * p.K + k;
          if (wide_out) {
            asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(q8[0]), "r"(q8[1]), "r"(q8[2]), "r"(q8[3]),
                         "r"(q8[4]), "r"(q8[5]), "r"(q8[6]), "r"(q8[7]) : "memory");
          } else {
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(q8[0], q8[1], q8[2], q8[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(q8[4], q8[5], q8[6], q8[7]);
          }
        }
        s_sf[(blk >> 2) * 512 + 16 * (rt & 31) + 4 * (rt >> 5) + (blk & 3)] = uint8_t(sf_code);
      }
      (void)q; (void)q8;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
      for (int j = 0; j < kWords; ++j) raw[u][j] = nxt[u][j];
    }
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
