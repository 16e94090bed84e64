/*
 * TEST INFRASTRUCTURE -- plain-C restatement of the reference's host block-scaled GEMM.
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may build,
 * load or call this file; the GPU library never does.
 *
 * Restates, from the reference tree (NVIDIA CUTLASS):
 *   - element decode / encode: include/cutlass/float_subbyte.h:81 (e2m1),
 *     include/cutlass/float8.h:1083-1259 (ue4m3, ue8m0), include/cutlass/exmy_base.h:640-845
 *     (round-to-nearest-even, saturate to the largest finite value);
 *   - the interleaved scale-factor layout: include/cutlass/detail/sm100_blockscaled_layout.hpp:49-114;
 *   - the GEMM itself: tools/util/include/cutlass/util/reference/host/gett.hpp:491-604
 *     (64x64 blocks, k sequential, a = float(A)*float(SFA), b = float(B)*float(SFB),
 *     acc = a*b + acc in fp32) and :690-800 (out = alpha*acc; out = beta*C + out);
 *   - NVFP4 output quantisation: gett.hpp:364-481.
 *
 * Multiply and add are rounded separately (build with -ffp-contract=off), as in the
 * compiled reference driver this file is pinned against (tests/test_oracle.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static const float kE2m1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

static float e4m3_value(uint32_t code) {
  uint32_t e = (code >> 3) & 0xF, m = code & 7;
  float v;
  if (e == 0xF && m == 7) return NAN;
  v = e == 0 ? ldexpf((float)m / 8.f, -6) : ldexpf(1.f + (float)m / 8.f, (int)e - 7);
  return (code & 0x80) ? -v : v;
}

/* fmt: 0 e2m1 (4-bit code), 1 e4m3, 2 ue4m3, 3 ue8m0 */
float bsg_oracle_decode(int fmt, uint32_t code) {
  switch (fmt) {
    case 0: return kE2m1[code & 0xF];
    case 1: return e4m3_value(code & 0xFF);
    case 2: return e4m3_value(code & 0x7F);
    default:
      code &= 0xFF;
      if (code == 0xFF) return NAN;
      return ldexpf(1.f, (int)code - 127);
  }
}

/* Round |x| to the nearest value of an ascending grid; ties go to the even index; saturate. */
static uint32_t nearest_even(float mag, const float* grid, int n) {
  int i;
  if (!(mag < grid[n - 1])) return (uint32_t)(n - 1);
  for (i = 1; i < n; ++i) {
    if (mag < grid[i]) {
      double lo = grid[i - 1], hi = grid[i], mid = 0.5 * (lo + hi);
      if ((double)mag > mid) return (uint32_t)i;
      if ((double)mag < mid) return (uint32_t)(i - 1);
      return (uint32_t)((i & 1) ? i - 1 : i);
    }
  }
  return (uint32_t)(n - 1);
}

static float g_e4m3_grid[127];
static int g_grid_ready = 0;
static void init_grid(void) {
  int c;
  if (g_grid_ready) return;
  for (c = 0; c < 127; ++c) g_e4m3_grid[c] = e4m3_value((uint32_t)c);
  g_grid_ready = 1;
}

uint32_t bsg_oracle_encode(int fmt, float x) {
  static const float e2m1_grid[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  uint32_t bits, sign;
  memcpy(&bits, &x, 4);
  sign = bits >> 31;
  init_grid();
  switch (fmt) {
    case 0:
      if (isnan(x)) return 0x7;
      return nearest_even(fabsf(x), e2m1_grid, 8) | (sign << 3);
    case 1:
      if (isnan(x)) return 0x7F;
      return nearest_even(fabsf(x), g_e4m3_grid, 127) | (sign << 7);
    case 2:
      if (isnan(x)) return 0x7F;
      return nearest_even(fabsf(x), g_e4m3_grid, 127);
    default: {
      uint32_t e = (bits >> 23) & 0xFF, m = bits & 0x7FFFFF;
      if (isnan(x) || isinf(x)) return 0xFF;
      if (m > 0 && e != 0xFE && !(e == 0 && m <= 0x00400000u)) e++;
      return e;
    }
  }
}

int64_t bsg_oracle_sf_offset(int64_t row, int64_t kblock, int64_t k_atoms) {
  return (row / 128) * (512 * k_atoms) + (kblock / 4) * 512 + 16 * (row % 32) + 4 * ((row % 128) / 32) + (kblock % 4);
}

static float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t bsg_oracle_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if (isnan(f)) return 0x7FC0;
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* Operand kinds: 0 NVFP4 (e2m1 data, ue4m3 scale per 16), 1 MXFP8 (e4m3, ue8m0 per 32), 2 MXFP4 (e2m1, ue8m0 per 32),
 * 3 mixed (A e4m3, B e2m1, both ue8m0 per 32: the reference's example 72c). */
static int kind_is_fp4(int kind, int is_b) { return kind == 0 || kind == 2 || (kind == 3 && is_b); }

/* value * scale for every element of a packed K-major operand -> rows x K floats */
static void expand_operand(int kind, int is_b, const uint8_t* data, const uint8_t* sf, int64_t rows, int64_t K, int64_t row_begin,
                           int64_t row_count, float* out) {
  const int vec = kind == 0 ? 16 : 32;
  const int fp4 = kind_is_fp4(kind, is_b);
  const int64_t kblocks = (K + vec - 1) / vec, k_atoms = (kblocks + 3) / 4;
  int64_t r, k;
  (void)rows;
  for (r = 0; r < row_count; ++r) {
    const int64_t row = row_begin + r;
    for (k = 0; k < K; ++k) {
      const uint8_t sc = sf[bsg_oracle_sf_offset(row, k / vec, k_atoms)];
      float v, s;
      if (fp4) {
        const uint8_t byte = data[row * (K / 2) + k / 2];
        v = kE2m1[(k & 1) ? (byte >> 4) : (byte & 0xF)];
      } else {
        v = e4m3_value(data[row * K + k]);
      }
      s = bsg_oracle_decode(kind == 0 ? 2 : 3, sc);
      out[r * K + k] = v * s;
    }
  }
}

/*
 * out[m, n] = alpha * sum_k a[m,k]*b[n,k] (+ beta * C[m,n]), fp32, for rows [m_begin, m_begin + m_count).
 * out is m_count x N.  C is bf16 bits with pitch ldc (may be NULL).  Returns 0 on success.
 */
/* Element-wise activations as the reference defines them (include/cutlass/epilogue/thread/activation.h:
 * ReLu :145 -- maximum with 0, NaN kept; GELU<float> :585; SiLu :452 with Sigmoid :408 and exp through the
 * host math library).  act: 0 identity, 1 ReLU, 2 GELU (erf form), 3 SiLU. */
float bsg_oracle_activation(int act, float x) {
  switch (act) {
    case 1: return x != x ? x : (x > 0.f ? x : 0.f);
    case 2: return (0.5f * x) * (1.0f + erff(x * 0.70710678118654752440f));
    case 3: return x * (1.0f / (1.0f + expf(-x)));
    default: return x;
  }
}

/* As bsg_oracle_gemm_rows, with the rest of the reference's epilogue (gett.hpp:714-761, in that order):
 * o = alpha * acc;  o = o + bias[n or m];  o = beta * C + o;  o = act(o).
 * bias_mode 0 none, 1 per column (N entries), 2 per row (M entries). */
int bsg_oracle_gemm_rows_epi(int kind, int64_t M, int64_t N, int64_t K, const uint8_t* A, const uint8_t* B, const uint8_t* SFA,
                             const uint8_t* SFB, const uint16_t* C, int64_t ldc, float alpha, float beta, const float* bias,
                             int bias_mode, int act, int64_t m_begin, int64_t m_count, float* out) {
  float* a = (float*)malloc(sizeof(float) * (size_t)(m_count * K));
  float* b = (float*)malloc(sizeof(float) * (size_t)(N * K));
  int64_t mb, nb;
  if (!a || !b) { free(a); free(b); return 1; }
  expand_operand(kind, 0, A, SFA, M, K, m_begin, m_count, a);
  {
    int64_t n0;
#pragma omp parallel for schedule(static)
    for (n0 = 0; n0 < N; n0 += 64) {
      const int64_t cnt = N - n0 < 64 ? N - n0 : 64;
      expand_operand(kind, 1, B, SFB, N, K, n0, cnt, b + n0 * K);
    }
  }
  {
    const int64_t mblocks = (m_count + 63) / 64, nblocks = (N + 63) / 64;
    int64_t blk;
#pragma omp parallel for schedule(dynamic) private(mb, nb)
    for (blk = 0; blk < mblocks * nblocks; ++blk) {
      float acc[64][64];
      float bt[64];
      int64_t k, i, j;
      int64_t mcnt, ncnt;
      mb = blk / nblocks;
      nb = blk % nblocks;
      mcnt = m_count - mb * 64 < 64 ? m_count - mb * 64 : 64;
      ncnt = N - nb * 64 < 64 ? N - nb * 64 : 64;
      for (i = 0; i < 64; ++i) for (j = 0; j < 64; ++j) acc[i][j] = 0.f;
      for (k = 0; k < K; ++k) {
        for (j = 0; j < 64; ++j) bt[j] = j < ncnt ? b[(nb * 64 + j) * K + k] : 0.f;
        for (i = 0; i < mcnt; ++i) {
          const float av = a[(mb * 64 + i) * K + k];
          for (j = 0; j < 64; ++j) acc[i][j] = av * bt[j] + acc[i][j];
        }
      }
      for (i = 0; i < mcnt; ++i) {
        const int64_t m = mb * 64 + i;
        for (j = 0; j < ncnt; ++j) {
          const int64_t n = nb * 64 + j;
          float o = alpha * acc[i][j];
          if (bias_mode == 1) o = o + bias[n];
          else if (bias_mode == 2) o = o + bias[m_begin + m];
          if (C) o = beta * bf16_to_f32(C[(m_begin + m) * ldc + n]) + o;
          out[m * N + n] = bsg_oracle_activation(act, o);
        }
      }
    }
  }
  free(a);
  free(b);
  return 0;
}

int bsg_oracle_gemm_rows(int kind, int64_t M, int64_t N, int64_t K, const uint8_t* A, const uint8_t* B, const uint8_t* SFA,
                         const uint8_t* SFB, const uint16_t* C, int64_t ldc, float alpha, float beta, int64_t m_begin,
                         int64_t m_count, float* out) {
  return bsg_oracle_gemm_rows_epi(kind, M, N, K, A, B, SFA, SFB, C, ldc, alpha, beta, NULL, 0, 0, m_begin, m_count, out);
}

/* Block-scaled quantisation of an fp32 (M x N) matrix along N, as the reference's epilogue and any
 * quantiser in front of the GEMM do it (tools/util/include/cutlass/util/reference/host/gett.hpp:364-481,
 * row-major branch :436-478): per row and per block of V elements, amax -> scale factor
 * SF = cvt(amax * (st * (1 / fp_max))) -> values cvt(x * min(st * (1 / float(SF)), FLT_MAX)).
 * kind 0: V = 16, SF ue4m3, values e2m1 packed two per byte (fp_max 6);
 * kind 1: V = 32, SF ue8m0 (conversion rounds up), values e4m3 (fp_max 448).
 * D is M x N/2 or M x N bytes; SFD is the interleaved scale-factor buffer (zero where nothing is written). */
void bsg_oracle_quant(int kind, const float* x, int64_t M, int64_t N, float st, uint8_t* D, uint8_t* SFD) {
  const int V = kind == 0 ? 16 : 32;
  const int sf_fmt = kind == 0 ? 2 : 3, d_fmt = kind == 0 ? 0 : 1;
  const float fp_max = kind == 0 ? 6.0f : 448.0f;
  const float scale_down = 1.0f / fp_max;
  const float st_scaled = st * scale_down;
  const int64_t nblocks = N / V, k_atoms = (nblocks + 3) / 4;
  int64_t m;
#pragma omp parallel for schedule(static)
  for (m = 0; m < M; ++m) {
    int64_t nb;
    for (nb = 0; nb < nblocks; ++nb) {
      const float* v = x + m * N + nb * V;
      float amax = 0.f, pv, qf, rcp, sc;
      uint32_t q;
      int j;
      /* maximum and minimum propagate NaN (maximum_with_nan_propogation / minimum_with_nan_propagation, gett.hpp:390,463):
       * one NaN in a block makes its scale factor and all of its values NaN codes (e2m1 has none: the largest value) */
      for (j = 0; j < V; ++j) { const float a = fabsf(v[j]); if (isnan(a) || isnan(amax)) amax = NAN; else if (a > amax) amax = a; }
      pv = amax * st_scaled;
      q = bsg_oracle_encode(sf_fmt, pv);
      SFD[bsg_oracle_sf_offset(m, nb, k_atoms)] = (uint8_t)q;
      qf = bsg_oracle_decode(sf_fmt, q);
      rcp = 1.0f / qf;
      sc = st * rcp;
      if (!isnan(sc) && sc > FLT_MAX) sc = FLT_MAX;
      if (kind == 0) {
        for (j = 0; j < V; j += 2) {
          const uint32_t lo = bsg_oracle_encode(d_fmt, v[j] * sc), hi = bsg_oracle_encode(d_fmt, v[j + 1] * sc);
          D[m * (N / 2) + nb * 8 + j / 2] = (uint8_t)(lo | (hi << 4));
        }
      } else {
        for (j = 0; j < V; ++j) D[m * N + nb * V + j] = (uint8_t)bsg_oracle_encode(d_fmt, v[j] * sc);
      }
    }
  }
}

/* NVFP4 re-quantisation of an fp32 (M x N) matrix: packed e2m1 D (M x N/2) and interleaved ue4m3 SFD. */
void bsg_oracle_quant_nvfp4(const float* x, int64_t M, int64_t N, float st, uint8_t* D, uint8_t* SFD) {
  bsg_oracle_quant(0, x, M, N, st, D, SFD);
}

void bsg_oracle_to_bf16(const float* x, int64_t n, uint16_t* out) {
  int64_t i;
  for (i = 0; i < n; ++i) out[i] = bsg_oracle_f32_to_bf16(x[i]);
}

/* Number of threads for the parallel regions the calling thread starts from now on (this library's and the
 * compiled reference's: they share the OpenMP runtime). */
void bsg_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int bsg_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
