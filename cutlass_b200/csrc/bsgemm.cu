// Host side of the C ABI declared in include/bsgemm.h: argument checks, TMA tensor
// maps, grid / cluster selection and kernel launch.  Takes the role of the reference's
// GemmUniversalAdapter (include/cutlass/gemm/device/gemm_universal_adapter.h:232-611).
//
// No allocation happens here; cuTensorMapEncodeTiled is resolved through the runtime
// (cudaGetDriverEntryPoint), so the library loads on machines without a driver.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <mutex>
#include <new>

#include "../../include/bsgemm.h"
#include "gemm_kernel.cuh"
#include "quant_kernel.cuh"

namespace {

thread_local char g_err[512] = "";

int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || p == nullptr) return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// Tensor maps are pure descriptions (address, extents, strides, box, swizzle), so one encoded for a given
// description stays valid for as long as that memory is used with that shape.  A small cache, guarded by a mutex,
// keeps the most recently used ones: a steady-state run encodes nothing.  (The reference encodes its
// descriptors in GemmUniversalAdapter::initialize and reuses them across run() calls, gemm_universal_adapter.h:313-375.)
struct MapKey {
  const void* base;
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  int32_t dtype, swizzle, l2;
};

// Set while the per-group maps of a pointer-array call are encoded: hundreds of one-off maps would only push the
// dense calls' entries out of the cache.
thread_local bool g_bypass_map_cache = false;

class MapCache {
 public:
  int32_t get(const MapKey& k, CUtensorMap* out) {
    if (!g_bypass_map_cache) {
      std::lock_guard<std::mutex> lock(mu_);
      for (int i = 0; i < kEntries; ++i) {
        if (used_[i] && memcmp(&keys_[i], &k, sizeof(MapKey)) == 0) {
          ticks_[i] = ++tick_;
          memcpy(out, &maps_[i], sizeof(CUtensorMap));
          return BSG_OK;
        }
      }
    }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(BSG_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[3] = {k.dims[0], k.dims[1], k.dims[2]};
    cuuint64_t strides[2] = {k.strides[0], k.strides[1]};
    cuuint32_t box[3] = {k.box[0], k.box[1], k.box[2]};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, static_cast<CUtensorMapDataType>(k.dtype), 3, const_cast<void*>(k.base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(k.swizzle),
                     static_cast<CUtensorMapL2promotion>(k.l2), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return fail(BSG_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (dims %llu x %llu x %llu, strides %llu, %llu bytes)", int(r),
                  (unsigned long long)k.dims[0], (unsigned long long)k.dims[1], (unsigned long long)k.dims[2],
                  (unsigned long long)k.strides[0], (unsigned long long)k.strides[1]);
    memcpy(out, &m, sizeof(CUtensorMap));
    if (g_bypass_map_cache) return BSG_OK;
    std::lock_guard<std::mutex> lock(mu_);
    int victim = 0;
    for (int i = 0; i < kEntries; ++i) {
      if (!used_[i]) { victim = i; break; }
      if (ticks_[i] < ticks_[victim]) victim = i;
    }
    keys_[victim] = k;
    memcpy(&maps_[victim], &m, sizeof(CUtensorMap));
    used_[victim] = true;
    ticks_[victim] = ++tick_;
    return BSG_OK;
  }

 private:
  static constexpr int kEntries = 64;
  std::mutex mu_;
  MapKey keys_[kEntries];
  CUtensorMap maps_[kEntries];
  bool used_[kEntries] = {};
  uint64_t ticks_[kEntries] = {};
  uint64_t tick_ = 0;
};

MapCache g_maps;

MapKey make_key(const void* base, int dtype, int swizzle, int l2, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s0, uint64_t s1,
                uint32_t b0, uint32_t b1, uint32_t b2) {
  MapKey k;
  memset(&k, 0, sizeof(k));     // padding bytes take part in the comparison
  k.base = base;
  k.dims[0] = d0; k.dims[1] = d1; k.dims[2] = d2;
  k.strides[0] = s0; k.strides[1] = s1;
  k.box[0] = b0; k.box[1] = b1; k.box[2] = b2;
  k.dtype = dtype; k.swizzle = swizzle; k.l2 = l2;
  return k;
}

// K-major byte matrices (batches x rows x row_bytes) with a row pitch and a batch stride, box = 128 bytes x box_rows,
// 128-byte swizzle.
int32_t make_operand_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t batches,
                         uint64_t pitch_bytes, uint64_t batch_stride_bytes, uint32_t box_rows) {
  return g_maps.get(make_key(base, CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             row_bytes, rows, batches, pitch_bytes, batch_stride_bytes, 128, box_rows, 1), map);
}

// Interleaved scale factors as (row_atoms, k_atoms, 512 bytes); box = box_row_atoms x box_k_atoms x 512 bytes.
int32_t make_sf_map(CUtensorMap* map, const void* base, uint64_t k_atoms, uint64_t row_atoms, uint32_t box_k_atoms,
                    uint32_t box_row_atoms) {
  return g_maps.get(make_key(base, CU_TENSOR_MAP_DATA_TYPE_UINT32, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             128, k_atoms, row_atoms, 512, 512 * k_atoms, 128, box_k_atoms, box_row_atoms), map);
}

// Output matrix for the epilogue's TMA stores, (batches x rows x cols); a box is 32 rows x 64 output columns:
// bf16: 128 bytes per row, 128-byte swizzle; e4m3: 64 bytes, 64-byte swizzle; packed e2m1: 32 bytes, no swizzle.
int32_t make_out_map(CUtensorMap* map, const void* base, int32_t out_kind, uint64_t cols, uint64_t rows, uint64_t batches,
                     uint64_t pitch_elems, uint64_t batch_stride_elems) {
  if (out_kind == BSG_OUT_F16)
    return g_maps.get(make_key(base, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                               cols, rows, batches, pitch_elems * 2, batch_stride_elems * 2, 64, 32, 1), map);
  if (out_kind == BSG_OUT_F32)      // 32 columns are 128 bytes: half a pair per store
    return g_maps.get(make_key(base, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                               cols, rows, batches, pitch_elems * 4, batch_stride_elems * 4, 32, 32, 1), map);
  if (out_kind == BSG_OUT_BF16)
    return g_maps.get(make_key(base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                               cols, rows, batches, pitch_elems * 2, batch_stride_elems * 2, 64, 32, 1), map);
  if (out_kind == BSG_OUT_MXFP8 || out_kind == BSG_OUT_E4M3 || out_kind == BSG_OUT_E5M2)
    return g_maps.get(make_key(base, CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                               cols, rows, batches, pitch_elems, batch_stride_elems, 64, 32, 1), map);
  return g_maps.get(make_key(base, CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                             cols / 2, rows, batches, pitch_elems / 2, batch_stride_elems / 2, 32, 32, 1), map);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Everything the launcher needs, independent of dense / grouped origin.
struct Problem {
  int32_t kind, out_kind;
  int32_t num_groups;
  int64_t rows_per_group;   // dense / batched
  int64_t total_rows;
  int64_t N, K;
  const void *A, *B, *SFA, *SFB, *C;
  void *D, *SFD;
  const int32_t* offsets;
  bool b_per_group;
  int64_t ldc, ldd;
  int64_t lda, ldb;                         // row pitch of A / B in elements
  int64_t bs_a, bs_b, bs_c, bs_d;           // batch strides in elements (dense / batched form only)
  int32_t use_pdl, scheduler, out_col_major;
  int32_t cluster[4];                       // cluster_m, cluster_n, fallback m, n (0 = default)
  float alpha, beta;
  const float *alpha_ptr, *beta_ptr, *norm_ptr;
  int32_t tile_n, cta_group, sm_count, raster_band;
  // gating (tensor parallel)
  const uint32_t* ready_flags;
  int32_t rows_per_flag;
  uint32_t flag_target;
  int32_t tile_m_rotate;
  // tensor parallel (TP kernel variant)
  bool tp;
  int32_t tp_world, tp_rank, tp_rows_per_shard, tp_ksplit, tp_push_in_kernel, tp_release_announce, tp_paced_push;
  uint32_t tp_epoch;
  const float* bias;
  const float* alpha_array;
  const float* beta_array;
  int32_t bias_mode, bias_group_stride, activation;
  uint32_t tp_ready_target; // a peer's buffer may be filled once the peer has launched this call number
  int32_t tp_parity;        // which of the two gathered buffers this call fills and reads (own rows always sit in buffer 0)
  int64_t tp_row_bytes, tp_sfa_rowatom_bytes;
  const uint8_t* tp_peer_a[8];
  const uint8_t* tp_peer_sfa[8];
  uint32_t* tp_peer_sync[8];
  int32_t* grid_ctas_out;     // receives the number of CTAs launched
  // GEMM + reduce-scatter (RS kernel variant)
  bool rs;
  int32_t rs_world, rs_rank, rs_slice_rows, rs_parity;
  uint32_t rs_epoch;
  const void* rs_recv;        // this rank's receive buffers
  void* rs_recv_left;         // receive buffers of rank - 1 (peer memory)
  uint32_t *rs_flags, *rs_flags_left, *rs_sync, *rs_sync_left, *rs_sync_right;
  // GEMM + all-reduce
  int32_t rs_allreduce, rs_out_half;
  uint32_t rs_done_target;
  const void* rs_out_maps;
  uint32_t* rs_peer_sync[8];
};

struct Plan {
  int32_t cta_group, tile_n, stages, smem_bytes;
  int64_t num_tiles;   // -1 if unknown on the host
};

int32_t validate(const Problem& q, Plan* plan) {
  if (q.kind < BSG_KIND_NVFP4 || q.kind > BSG_KIND_MXFP8_MXFP4) return fail(BSG_ERR_NOT_SUPPORTED, "unknown operand kind %d", q.kind);
  if (q.out_kind < BSG_OUT_BF16 || q.out_kind > BSG_OUT_E5M2) return fail(BSG_ERR_NOT_SUPPORTED, "unknown output kind %d", q.out_kind);
  const bool quantised_out = q.out_kind == BSG_OUT_NVFP4 || q.out_kind == BSG_OUT_MXFP8;
  if (q.rs && q.out_kind != BSG_OUT_BF16) return fail(BSG_ERR_NOT_SUPPORTED, "the reduce-scatter GEMM writes bf16");
  if ((q.out_kind >= BSG_OUT_F16 || q.out_col_major) &&
      (q.kind > BSG_KIND_MXFP8 || q.tp || q.scheduler != BSG_SCHED_STATIC || (q.cta_group != 0 && q.cta_group != 2)))
    return fail(BSG_ERR_NOT_SUPPORTED, "fp16 / fp32 / e4m3 / e5m2 outputs and column-major quantised outputs are available for NVFP4 and MXFP8 operands with cta_group 2 and the static scheduler, on one GPU");
  if (q.num_groups < 1 || q.num_groups > BSG_MAX_GROUPS) return fail(BSG_ERR_INVALID_PROBLEM, "group / batch count %d outside [1, %d]", q.num_groups, BSG_MAX_GROUPS);
  if (q.N < 1 || q.K < 1 || q.total_rows < 0) return fail(BSG_ERR_INVALID_PROBLEM, "extents must be positive (rows=%lld N=%lld K=%lld)", (long long)q.total_rows, (long long)q.N, (long long)q.K);
  if (q.total_rows > 0x7FFFFFFF / 2 || q.N > 0x7FFFFFFF / 2 || q.K > 0x7FFFFFFF / 2) return fail(BSG_ERR_INVALID_PROBLEM, "extent exceeds 2^30");
  // 16 bytes of K per row; the mixed kind expands B's e2m1 values in blocks of 128 on their way into shared memory
  const int64_t k_align = q.kind == BSG_KIND_MXFP8 ? 16 : q.kind == BSG_KIND_MXFP8_MXFP4 ? 128 : 32;
  if (q.K % k_align != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "K=%lld must be a multiple of %lld", (long long)q.K, (long long)k_align);
  if (!q.A || !q.B || !q.SFA || !q.SFB || !q.D) return fail(BSG_ERR_INVALID_PROBLEM, "A, B, SFA, SFB and D must be non-null");
  if (!aligned16(q.A) || !aligned16(q.B) || !aligned16(q.D) || (q.C && !aligned16(q.C)))
    return fail(BSG_ERR_MISALIGNED_OPERAND, "A, B, C and D must be 16-byte aligned");
  if (!aligned16(q.SFA) || !aligned16(q.SFB)) return fail(BSG_ERR_MISALIGNED_OPERAND, "scale-factor tensors must be 16-byte aligned");
  if (q.out_col_major) {
    // column-major quantised output: D is (N, M) with M contiguous, scale factors along M
    if (!quantised_out) return fail(BSG_ERR_NOT_SUPPORTED, "the column-major layout is for quantised outputs");
    if (q.offsets || q.num_groups != 1 || q.tp || q.rs) return fail(BSG_ERR_NOT_SUPPORTED, "the column-major output layout is for the dense, unbatched GEMM");
    if (!q.SFD || (q.out_kind == BSG_OUT_NVFP4 && !q.norm_ptr)) return fail(BSG_ERR_INVALID_PROBLEM, "quantised output needs SFD (and norm_constant for NVFP4)");
    if (q.rows_per_group % 32 != 0 || q.ldd % 32 != 0 || q.ldd < q.rows_per_group)
      return fail(BSG_ERR_MISALIGNED_OPERAND, "column-major output needs M %% 32 == 0 and ldd (the pitch of a column, >= M) %% 32 == 0");
  } else if (q.out_kind == BSG_OUT_BF16 || q.out_kind == BSG_OUT_F16) {
    if (q.N % 8 != 0 || q.ldd % 8 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "bf16 / fp16 output needs N and ldd to be multiples of 8");
  } else if (q.out_kind == BSG_OUT_F32) {
    if (q.N % 4 != 0 || q.ldd % 4 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "fp32 output needs N and ldd to be multiples of 4");
  } else if (q.out_kind == BSG_OUT_E4M3 || q.out_kind == BSG_OUT_E5M2) {
    if (q.N % 16 != 0 || q.ldd % 16 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "e4m3 / e5m2 output needs N and ldd to be multiples of 16");
  } else if (q.out_kind == BSG_OUT_MXFP8) {
    if (!q.SFD) return fail(BSG_ERR_INVALID_PROBLEM, "MXFP8 output needs SFD");
    if (q.N % 32 != 0 || q.ldd % 16 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "MXFP8 output needs N %% 32 == 0 and ldd %% 16 == 0");
  } else {
    if (!q.SFD || !q.norm_ptr) return fail(BSG_ERR_INVALID_PROBLEM, "NVFP4 output needs SFD and norm_constant");
    if (q.N % 16 != 0 || q.ldd % 32 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "NVFP4 output needs N %% 16 == 0 and ldd %% 32 == 0");
  }
  if (q.bias_mode < BSG_BIAS_NONE || q.bias_mode > BSG_BIAS_PER_ROW) return fail(BSG_ERR_NOT_SUPPORTED, "unknown bias mode %d", q.bias_mode);
  if (q.bias_mode != BSG_BIAS_NONE) {
    if (!q.bias) return fail(BSG_ERR_INVALID_PROBLEM, "bias mode %d needs a bias vector", q.bias_mode);
    if (!aligned16(q.bias)) return fail(BSG_ERR_MISALIGNED_OPERAND, "bias must be 16-byte aligned");
    if (q.bias_mode == BSG_BIAS_PER_COLUMN && q.N % 4 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "per-column bias needs N %% 4 == 0");
    if (q.bias_mode == BSG_BIAS_PER_ROW && q.offsets) return fail(BSG_ERR_NOT_SUPPORTED, "per-row bias is not available for grouped GEMM");
  }
  if (q.activation < BSG_ACT_IDENTITY || q.activation > BSG_ACT_SILU) return fail(BSG_ERR_NOT_SUPPORTED, "unknown activation %d", q.activation);
  if (q.C && (q.ldc % 8 != 0)) return fail(BSG_ERR_MISALIGNED_OPERAND, "ldc must be a multiple of 8");
  if ((!q.out_col_major && q.ldd < q.N) || (q.C && q.ldc < q.N)) return fail(BSG_ERR_INVALID_PROBLEM, "row pitch smaller than N");
  if (q.lda < q.K || q.ldb < q.K) return fail(BSG_ERR_INVALID_PROBLEM, "lda / ldb smaller than K");
  if (q.lda % k_align != 0 || q.ldb % k_align != 0)
    return fail(BSG_ERR_MISALIGNED_OPERAND, "lda=%lld and ldb=%lld must be multiples of %lld (16-byte rows)", (long long)q.lda, (long long)q.ldb, (long long)k_align);
  if (!q.offsets && q.num_groups > 1) {
    if (q.bs_a % k_align != 0 || q.bs_b % k_align != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "batch strides of A and B must be multiples of %lld elements", (long long)k_align);
    const int64_t d_align = q.out_kind == BSG_OUT_F32 ? 4 : (q.out_kind == BSG_OUT_E4M3 || q.out_kind == BSG_OUT_E5M2) ? 16 : !quantised_out ? 8 : q.out_kind == BSG_OUT_MXFP8 ? 16 : 32;
    if (q.bs_d % d_align != 0 || (q.C && q.bs_c % 8 != 0)) return fail(BSG_ERR_MISALIGNED_OPERAND, "batch strides of C and D must keep every matrix 16-byte aligned");
    if (q.bs_a < 0 || q.bs_b < 0 || q.bs_c < 0 || q.bs_d < q.rows_per_group * q.ldd) return fail(BSG_ERR_INVALID_PROBLEM, "negative batch stride, or output matrices that overlap");
  }
  if (q.use_pdl != 0 && q.use_pdl != 1) return fail(BSG_ERR_INVALID_PROBLEM, "use_pdl must be 0 or 1");
  if (q.scheduler != BSG_SCHED_STATIC && q.scheduler != BSG_SCHED_DYNAMIC) return fail(BSG_ERR_NOT_SUPPORTED, "unknown scheduler %d", q.scheduler);
  if (q.beta != 0.0f && !q.C && !q.beta_ptr) return fail(BSG_ERR_INVALID_PROBLEM, "beta != 0 needs C");
  if (q.beta_array && !q.C) return fail(BSG_ERR_INVALID_PROBLEM, "per-group beta needs C");
  int32_t cg = q.cta_group == 0 ? 2 : q.cta_group;
  int32_t tn = q.tile_n == 0 ? (q.N > 128 ? 256 : 128) : q.tile_n;
  if (cg != 1 && cg != 2) return fail(BSG_ERR_NOT_SUPPORTED, "cta_group must be 1 or 2");
  if (tn != 64 && tn != 128 && tn != 192 && tn != 256) return fail(BSG_ERR_NOT_SUPPORTED, "tile_n must be 64, 128, 192 or 256");
  if ((tn == 64 || tn == 192) && (q.kind > BSG_KIND_MXFP8 || cg != 2 || q.scheduler != BSG_SCHED_STATIC || q.tp || q.rs || q.out_kind >= BSG_OUT_F16 || q.out_col_major))
    return fail(BSG_ERR_NOT_SUPPORTED, "tiles of 64 and 192 columns are available for NVFP4 and MXFP8 operands with cta_group 2, the static scheduler and bf16 or re-quantised row-major output, on one GPU");
  // Cluster shapes: the cluster is the CTA group of one MMA, there is nothing larger to prefer or to fall back to.
  for (int i = 0; i < 4; i += 2) {
    if ((q.cluster[i] != 0 || q.cluster[i + 1] != 0) && !(q.cluster[i] == cg && q.cluster[i + 1] == 1))
      return fail(BSG_ERR_NOT_SUPPORTED, "%scluster shape %d x %d is not available: this configuration runs clusters of %d x 1",
                  i ? "fallback " : "", q.cluster[i], q.cluster[i + 1], cg);
  }
  if (q.kind >= BSG_KIND_MXFP4 && (cg != 2 || q.scheduler != BSG_SCHED_STATIC || q.tp || q.rs))
    return fail(BSG_ERR_NOT_SUPPORTED, "MXFP4 and mixed MXFP8 x MXFP4 operands run with cta_group 2 and the static scheduler only");
  if (q.kind == BSG_KIND_MXFP8_MXFP4 && (reinterpret_cast<uintptr_t>(q.B) & 31u) != 0)
    return fail(BSG_ERR_MISALIGNED_OPERAND, "B of the mixed kind must be 32-byte aligned");
  if (q.scheduler == BSG_SCHED_DYNAMIC && (q.tp || cg != 2)) return fail(BSG_ERR_NOT_SUPPORTED, "the dynamic scheduler needs cta_group 2 and is not available for the tensor-parallel GEMM");
  plan->cta_group = cg;
  plan->tile_n = tn;
  if (q.offsets) {
    plan->num_tiles = -1;
  } else {
    const int64_t tile_m = 128 * cg;
    plan->num_tiles = int64_t(q.num_groups) * ((q.rows_per_group + tile_m - 1) / tile_m) * ((q.N + tn - 1) / tn);
  }
  return BSG_OK;
}

// Per kernel instantiation and device: the dynamic shared-memory limit is raised once, and the number of clusters
// that can be resident at the same time is asked once (the grid never exceeds it: the roles of a persistent kernel
// wait on one another across CTAs only inside a cluster, but the tensor-parallel variant also waits for rows that
// the push warps of OTHER CTAs of a peer deliver, so every CTA of a launch must be resident).
struct KernelSetup {
  std::mutex mu;
  bool done[64] = {};
  int max_clusters[64] = {};
};

template <int KIND, int CG, int BN, bool TP, bool DYN, bool RS, bool PTR = false, bool OUTX = false>
int32_t kernel_setup(int dev, int* max_clusters) {
  using Cf = bsg::Cfg<KIND, CG, BN, TP>;
  static KernelSetup ks;
  if (dev < 0 || dev >= 64) return fail(BSG_ERR_NOT_SUPPORTED, "device ordinal %d is outside [0, 64)", dev);
  std::lock_guard<std::mutex> lock(ks.mu);
  if (!ks.done[dev]) {
    auto kernel = bsg::bsg_gemm_kernel<KIND, CG, BN, TP, DYN, RS, PTR, OUTX>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cf::kSmemBytes);
    if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(unsigned(CG) * 1024u, 1, 1);
    cfg.blockDim = dim3(TP ? 224 : 192, 1, 1);
    cfg.dynamicSmemBytes = Cf::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
    if (e != cudaSuccess || n < 1) { cudaGetLastError(); n = 0; }     // unknown: do not clamp
    ks.max_clusters[dev] = n;
    ks.done[dev] = true;
  }
  *max_clusters = ks.max_clusters[dev];
  return BSG_OK;
}

template <int KIND, int CG, int BN, bool TP = false, bool DYN = false, bool RS = false, bool OUTX = false>
int32_t launch(const Problem& q, const Plan& plan, uint32_t* status, cudaStream_t stream, int sm_count, int dev, bool dry) {
  using Cf = bsg::Cfg<KIND, CG, BN, TP>;
  if (dry) return BSG_OK;
  const bool a_fp4 = bsg::kind_packs_fp4(KIND), b_fp4 = KIND != bsg::kKindMxfp8;     // two values per byte in global memory
  const int64_t ka_bytes = a_fp4 ? q.K / 2 : q.K, kb_bytes = b_fp4 ? q.K / 2 : q.K;
  const int64_t k_atoms = ((q.K + Cf::kSfVec - 1) / Cf::kSfVec + 3) / 4;
  const int64_t n_atoms = (q.N + 127) / 128;
  const int64_t b_groups = q.b_per_group ? q.num_groups : 1;
  const bool batched = !q.offsets && !TP;          // dense / batched form: rows are addressed per batch entry
  int64_t sfa_row_atoms;
  if (q.offsets) sfa_row_atoms = q.total_rows / 128 + q.num_groups;   // upper bound; fetches are clamped per group
  else sfa_row_atoms = int64_t(q.num_groups) * ((q.rows_per_group + 127) / 128);
  const int64_t lda_bytes = a_fp4 ? q.lda / 2 : q.lda, ldb_bytes = b_fp4 ? q.ldb / 2 : q.ldb;
  const int64_t bsa_bytes = a_fp4 ? q.bs_a / 2 : q.bs_a, bsb_bytes = b_fp4 ? q.bs_b / 2 : q.bs_b;

  CUtensorMap tmA, tmB, tmSFA, tmSFB, tmD, tmDpeer;
  int32_t rc;
  // Rows of the A and D maps: one batch entry (batched form), all groups (grouped), or the two gathered buffers of
  // the tensor-parallel GEMM, which lie back to back.
  const uint64_t map_rows = batched ? uint64_t(q.rows_per_group) : uint64_t(TP ? 2 * q.total_rows : q.total_rows);
  const uint64_t map_batches = batched ? uint64_t(q.num_groups) : 1u;
  // Reduce-scatter: D is this rank's slice of the result; the other stages store into rank - 1's receive buffers
  // (two halves of world - 1 slices each, N columns wide).
  const uint64_t d_rows = RS ? uint64_t(q.rs_slice_rows) : batched ? uint64_t(q.rows_per_group) : uint64_t(q.total_rows);
  if (q.out_col_major)     // stored as its transpose (N rows of M values); the kernel writes it with plain stores, the map only describes it
    rc = make_out_map(&tmD, q.D, q.out_kind, uint64_t(q.rows_per_group), uint64_t(q.N), 1, uint64_t(q.ldd), uint64_t(q.N) * uint64_t(q.ldd));
  else
    rc = make_out_map(&tmD, q.D, q.out_kind, uint64_t(q.N), d_rows, map_batches, uint64_t(q.ldd),
                      uint64_t(batched && q.num_groups > 1 ? q.bs_d : d_rows * q.ldd));
  if (rc != BSG_OK) return rc;
  tmDpeer = tmD;
  if (RS && q.rs_world > 1) {
    const uint64_t peer_rows = 2ull * uint64_t(q.rs_world - 1) * uint64_t(q.rs_slice_rows);
    if ((rc = make_out_map(&tmDpeer, q.rs_recv_left, BSG_OUT_BF16, uint64_t(q.N), peer_rows, 1, uint64_t(q.N), peer_rows * uint64_t(q.N))) != BSG_OK) return rc;
  }
  if ((rc = make_operand_map(&tmA, q.A, uint64_t(ka_bytes), map_rows, map_batches, uint64_t(lda_bytes),
                             uint64_t(batched && q.num_groups > 1 ? bsa_bytes : int64_t(map_rows) * lda_bytes), Cf::kCtaM)) != BSG_OK) return rc;
  if (KIND == bsg::kKindMxfp8Mxfp4) {
    // B is packed e2m1 in global memory; the TMA engine spreads it into the form kind::mxf8f6f4 reads (16 values in
    // 8 bytes followed by 8 bytes of padding).  Extents and the box are counted in elements, strides in bytes.
    rc = g_maps.get(make_key(q.B, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             uint64_t(q.K), uint64_t(q.N), uint64_t(b_groups), uint64_t(ldb_bytes),
                             uint64_t(b_groups > 1 ? bsb_bytes : q.N * ldb_bytes), 128, Cf::kBRowsCta, 1), &tmB);
  } else {
    rc = make_operand_map(&tmB, q.B, uint64_t(kb_bytes), uint64_t(q.N), uint64_t(b_groups), uint64_t(ldb_bytes),
                          uint64_t(b_groups > 1 ? bsb_bytes : q.N * ldb_bytes), Cf::kBRowsCta);
  }
  if (rc != BSG_OK) return rc;
  if ((rc = make_sf_map(&tmSFA, q.SFA, k_atoms, TP ? 2 * sfa_row_atoms : sfa_row_atoms, Cf::kKAtoms, 1)) != BSG_OK) return rc;
  if ((rc = make_sf_map(&tmSFB, q.SFB, k_atoms, b_groups * n_atoms, Cf::kKAtoms, Cf::kSfbAtoms)) != BSG_OK) return rc;

  bsg::GemmParams p;
  memset(&p, 0, sizeof(p));
  p.num_groups = q.num_groups;
  p.rows_per_group = int32_t(q.rows_per_group);
  p.total_rows = int32_t(q.total_rows);
  p.N = int32_t(q.N);
  p.K = int32_t(q.K);
  p.offsets = q.offsets;
  p.b_per_group = q.b_per_group ? 1 : 0;
  p.sfb_atoms_per_group = q.b_per_group ? int32_t(n_atoms) : 0;
  p.batched = batched ? 1 : 0;
  p.batch_stride_c = batched ? q.bs_c : 0;
  p.batch_stride_d = batched ? q.bs_d : 0;
  p.tiles_n = int32_t((q.N + BN - 1) / BN);
  p.raster_band = q.raster_band > 0 ? q.raster_band : 16;
  p.out_kind = q.out_kind;
  p.out_col_major = q.out_col_major;
  p.alpha_array = q.alpha_array; p.beta_array = q.beta_array;
  p.bias = q.bias; p.bias_mode = q.bias_mode; p.bias_group_stride = q.bias_group_stride; p.activation = q.activation;
  p.C = static_cast<const __nv_bfloat16*>(q.C);
  p.D = q.D;
  p.SFD = static_cast<uint8_t*>(q.SFD);
  p.ldc = q.ldc;
  p.ldd = q.ldd;
  p.alpha = q.alpha;
  p.beta = q.beta;
  p.alpha_ptr = q.alpha_ptr;
  p.beta_ptr = q.beta_ptr;
  p.norm_ptr = q.norm_ptr;
  p.status = status;
  p.ready_flags = q.ready_flags;
  p.rows_per_flag = q.rows_per_flag;
  p.flag_target = q.flag_target;
  p.tile_m_rotate = q.tile_m_rotate;
  p.split_tail = 1;
  if (RS) {
    const int32_t tiles_per_slice = q.rs_slice_rows / (128 * CG);
    p.rs_world = q.rs_world;
    p.rs_tiles_per_slice = tiles_per_slice;
    p.rs_slice_rows = q.rs_slice_rows;
    p.rs_parity_rows = q.rs_parity ? (q.rs_world - 1) * q.rs_slice_rows : 0;
    p.rs_flag_target = uint32_t(4 * CG) * ((q.rs_epoch + 1u) >> 1);
    p.rs_ready_target = q.rs_epoch - 1u;
    p.rs_epoch = q.rs_epoch;
    p.rs_recv = static_cast<const __nv_bfloat16*>(q.rs_recv);
    p.rs_flags = q.rs_flags; p.rs_flags_left = q.rs_flags_left;
    p.rs_sync = q.rs_sync; p.rs_sync_left = q.rs_sync_left; p.rs_sync_right = q.rs_sync_right;
    p.rs_allreduce = q.rs_allreduce; p.rs_rank = q.rs_rank; p.rs_out_half = q.rs_out_half; p.rs_done_target = q.rs_done_target;
    p.rs_out_maps = static_cast<const CUtensorMap*>(q.rs_out_maps);
    for (int i = 0; i < 8; ++i) p.rs_peer_sync[i] = q.rs_peer_sync[i];
    p.split_tail = 0;
    // the walk starts at slice rank + 1 and ends at the rank's own slice; a band of the raster never straddles slices
    p.tile_m_rotate = ((q.rs_rank + 1) % q.rs_world) * tiles_per_slice;
    int32_t band = p.raster_band;
    while (tiles_per_slice % band != 0) band >>= 1;
    p.raster_band = band < 1 ? 1 : band;
  }
  if (TP) {
    p.tp_world = q.tp_world; p.tp_rank = q.tp_rank; p.tp_rows_per_shard = q.tp_rows_per_shard; p.tp_ksplit = q.tp_ksplit; p.tp_push_in_kernel = q.tp_push_in_kernel;
    p.tp_epoch = q.tp_epoch;
    p.tp_release_announce = q.tp_release_announce;
    p.tp_paced_push = q.tp_paced_push;
    p.tp_ready_target = q.tp_ready_target;
    p.tp_remote_row_offset = q.tp_parity ? int32_t(q.total_rows) : 0;
    p.tp_row_bytes = q.tp_row_bytes; p.tp_sfa_rowatom_bytes = q.tp_sfa_rowatom_bytes;
    for (int i = 0; i < 8; ++i) { p.tp_peer_a[i] = q.tp_peer_a[i]; p.tp_peer_sfa[i] = q.tp_peer_sfa[i]; p.tp_peer_sync[i] = q.tp_peer_sync[i]; }
  }
#ifdef BSG_PROFILE
  { const char* dbg = getenv("BSG_DEBUG_FLAGS"); p.debug_flags = dbg ? atoi(dbg) : 0; }
#endif

  int max_clusters = 0;
  if ((rc = kernel_setup<KIND, CG, BN, TP, DYN, RS, false, OUTX>(dev, &max_clusters)) != BSG_OK) return rc;
  auto kernel = bsg::bsg_gemm_kernel<KIND, CG, BN, TP, DYN, RS, false, OUTX>;

  int64_t clusters = sm_count / CG;
  if (max_clusters > 0 && clusters > max_clusters) clusters = max_clusters;
  if (plan.num_tiles >= 0 && plan.num_tiles < clusters) clusters = plan.num_tiles;
  if (DYN) {
    // One cluster per output tile: the hardware starts as many as fit, and every running cluster takes over the
    // tiles of clusters that have not started (the launch itself is the work queue).  Grouped problems only know an
    // upper bound of their tile count here; the kernel skips the surplus ids.
    const int64_t tile_m = 128 * CG;
    clusters = plan.num_tiles >= 0 ? plan.num_tiles : (q.total_rows / tile_m + q.num_groups) * ((q.N + BN - 1) / BN);
    if (clusters > 0x3FFFFFFF / CG) return fail(BSG_ERR_INVALID_PROBLEM, "too many tiles for one launch");
  }
  if (clusters < 1) clusters = 1;

  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(unsigned(clusters * CG), 1, 1);
  cfg.blockDim = dim3(TP ? 224 : 192, 1, 1);
  if (q.grid_ctas_out) *q.grid_ctas_out = int32_t(clusters * CG);
  cfg.dynamicSmemBytes = Cf::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (q.use_pdl && !TP) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmSFA, tmSFB, tmD, tmDpeer, p);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  return BSG_OK;
}

template <int KIND>
int32_t dispatch_shape(const Problem& q, const Plan& plan, uint32_t* status, cudaStream_t s, int sm, int dev, bool dry) {
  if (q.out_kind >= BSG_OUT_F16 || q.out_col_major) {      // checked in validate: cta_group 2, static scheduler, one GPU
    return plan.tile_n == 256 ? launch<KIND, 2, 256, false, false, false, true>(q, plan, status, s, sm, dev, dry)
                              : launch<KIND, 2, 128, false, false, false, true>(q, plan, status, s, sm, dev, dry);
  }
  if (q.rs) {
    if (plan.cta_group != 2 || plan.tile_n != 256) return fail(BSG_ERR_NOT_SUPPORTED, "the reduce-scatter GEMM runs 256 x 256 tiles (cta_group 2)");
    return launch<KIND, 2, 256, false, false, true>(q, plan, status, s, sm, dev, dry);
  }
  if (q.tp) {
    if (plan.cta_group != 2) return fail(BSG_ERR_NOT_SUPPORTED, "the tensor-parallel GEMM needs cta_group 2");
    return plan.tile_n == 256 ? launch<KIND, 2, 256, true>(q, plan, status, s, sm, dev, dry) : launch<KIND, 2, 128, true>(q, plan, status, s, sm, dev, dry);
  }
  if (plan.cta_group == 2 && q.scheduler == BSG_SCHED_DYNAMIC) {
    return plan.tile_n == 256 ? launch<KIND, 2, 256, false, true>(q, plan, status, s, sm, dev, dry)
                              : launch<KIND, 2, 128, false, true>(q, plan, status, s, sm, dev, dry);
  }
  if (plan.cta_group == 2) {
    if (plan.tile_n == 64) return launch<KIND, 2, 64>(q, plan, status, s, sm, dev, dry);
    if (plan.tile_n == 192) return launch<KIND, 2, 192>(q, plan, status, s, sm, dev, dry);
    return plan.tile_n == 256 ? launch<KIND, 2, 256>(q, plan, status, s, sm, dev, dry) : launch<KIND, 2, 128>(q, plan, status, s, sm, dev, dry);
  }
  return plan.tile_n == 256 ? launch<KIND, 1, 256>(q, plan, status, s, sm, dev, dry) : launch<KIND, 1, 128>(q, plan, status, s, sm, dev, dry);
}

template <int KIND, int CG, int BN>
void fill_caps_for(bsg_caps* caps) {
  using Cf = bsg::Cfg<KIND, CG, BN>;
  caps->tile_m = Cf::kTileM;
  caps->tile_n = BN;
  caps->tile_k = Cf::kTileK;
  caps->cta_group = CG;
  caps->stages = Cf::kStages;
  caps->smem_bytes = Cf::kSmemBytes;
}

void fill_caps(const Problem& q, const Plan& plan, bsg_caps* caps) {
  if (!caps) return;
  const bool fp4 = q.kind == BSG_KIND_NVFP4 || q.kind == BSG_KIND_MXFP4;     // the same tile extents and stage count
  if (plan.cta_group == 2 && plan.tile_n == 64) fp4 ? fill_caps_for<0, 2, 64>(caps) : fill_caps_for<1, 2, 64>(caps);
  else if (plan.cta_group == 2 && plan.tile_n == 192) fp4 ? fill_caps_for<0, 2, 192>(caps) : fill_caps_for<1, 2, 192>(caps);
  else if (plan.cta_group == 2 && plan.tile_n == 256) fp4 ? fill_caps_for<0, 2, 256>(caps) : fill_caps_for<1, 2, 256>(caps);
  else if (plan.cta_group == 2) fp4 ? fill_caps_for<0, 2, 128>(caps) : fill_caps_for<1, 2, 128>(caps);
  else if (plan.tile_n == 256) fp4 ? fill_caps_for<0, 1, 256>(caps) : fill_caps_for<1, 1, 256>(caps);
  else fp4 ? fill_caps_for<0, 1, 128>(caps) : fill_caps_for<1, 1, 128>(caps);
  caps->num_tiles = plan.num_tiles;
}

int32_t run_problem(const Problem& q, void* workspace, size_t ws_bytes, void* stream_v) {
  Plan plan;
  int32_t rc = validate(q, &plan);
  if (rc != BSG_OK) return rc;
  if (!workspace) return fail(BSG_ERR_WORKSPACE_NULL, "workspace is null");
  if (ws_bytes < 16) return fail(BSG_ERR_WORKSPACE_NULL, "workspace smaller than 16 bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 3u) != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "workspace must be 4-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  int dev = 0, major = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (major != 10) return fail(BSG_ERR_ARCH_MISMATCH, "device compute capability %d.x is not sm_100", major);
  if (q.sm_count > 0 && q.sm_count < sms) sms = q.sm_count;
  if (q.total_rows == 0) return BSG_OK;   // nothing to compute

  uint32_t* status = static_cast<uint32_t*>(workspace);
  if (q.kind == BSG_KIND_NVFP4) return dispatch_shape<0>(q, plan, status, stream, sms, dev, false);
  if (q.kind == BSG_KIND_MXFP8) return dispatch_shape<1>(q, plan, status, stream, sms, dev, false);
  // MXFP4 and the mixed kind: 2-CTA tiles, static scheduler (checked in validate)
  if (q.kind == BSG_KIND_MXFP4)
    return plan.tile_n == 256 ? launch<2, 2, 256>(q, plan, status, stream, sms, dev, false) : launch<2, 2, 128>(q, plan, status, stream, sms, dev, false);
  return plan.tile_n == 256 ? launch<3, 2, 256>(q, plan, status, stream, sms, dev, false) : launch<3, 2, 128>(q, plan, status, stream, sms, dev, false);
}


// ------------------------------------------------------------------------------ pointer-array grouped form
constexpr size_t kPtrTableOffset = 8192;      // the group table starts here in the workspace (the status word sits at 0)

struct PtrGroup {
  int64_t M, N, K, lda, ldb, ldc, ldd;
  const void *A, *B, *SFA, *SFB, *C;
  void *D, *SFD;
};

PtrGroup ptr_group(const bsg_ptr_array_args* a, int g) {
  PtrGroup r;
  r.M = a->problem_sizes[3 * g + 0]; r.N = a->problem_sizes[3 * g + 1]; r.K = a->problem_sizes[3 * g + 2];
  r.lda = a->lda ? a->lda[g] : r.K; r.ldb = a->ldb ? a->ldb[g] : r.K;
  r.ldc = a->ldc ? a->ldc[g] : r.N; r.ldd = a->ldd ? a->ldd[g] : r.N;
  r.A = a->A[g]; r.B = a->B[g]; r.SFA = a->SFA[g]; r.SFB = a->SFB[g];
  r.C = a->C ? a->C[g] : nullptr;
  r.D = a->D[g];
  r.SFD = a->SFD ? a->SFD[g] : nullptr;
  return r;
}

// What bsg_ptr_array_initialize left in a workspace, remembered on the host so that a run can check that it
// launches against a table made for the same problem.
struct PtrTableInfo {
  int32_t kind, out_kind, num_groups, tile_n;
  int64_t total_tiles, total_rows;
  uint64_t sizes_hash;
};
std::mutex g_ptr_tables_mutex;
constexpr int kPtrTables = 256;
struct { const void* ws; PtrTableInfo info; } g_ptr_tables[kPtrTables];
int g_ptr_tables_next = 0;

uint64_t hash_sizes(const int32_t* v, int n) {
  uint64_t h = 1469598103934665603ull;
  for (int i = 0; i < n; ++i) { h ^= uint64_t(uint32_t(v[i])); h *= 1099511628211ull; }
  return h;
}

// Checks the call-level fields and every group (the dense rules, group by group); returns the tile width and counts.
int32_t ptr_array_check(const bsg_ptr_array_args* a, PtrTableInfo* info) {
  if (!a) return fail(BSG_ERR_INVALID_PROBLEM, "args is null");
  if (a->kind != BSG_KIND_NVFP4 && a->kind != BSG_KIND_MXFP8) return fail(BSG_ERR_NOT_SUPPORTED, "the pointer-array form takes NVFP4 or MXFP8 operands (kind %d)", a->kind);
  if (a->num_groups < 1 || a->num_groups > BSG_MAX_GROUPS) return fail(BSG_ERR_INVALID_PROBLEM, "group count %d outside [1, %d]", a->num_groups, BSG_MAX_GROUPS);
  if (!a->problem_sizes || !a->A || !a->B || !a->SFA || !a->SFB || !a->D) return fail(BSG_ERR_INVALID_PROBLEM, "problem_sizes, A, B, SFA, SFB and D arrays must be non-null");
  if ((a->out_kind == BSG_OUT_NVFP4 || a->out_kind == BSG_OUT_MXFP8) && !a->SFD) return fail(BSG_ERR_INVALID_PROBLEM, "quantised output needs the SFD array");
  if (a->tile_n != 0 && a->tile_n != 128 && a->tile_n != 256) return fail(BSG_ERR_NOT_SUPPORTED, "tile_n must be 0, 128 or 256");
  if (a->use_pdl != 0 && a->use_pdl != 1) return fail(BSG_ERR_INVALID_PROBLEM, "use_pdl must be 0 or 1");
  if ((a->beta != 0.0f || a->beta_array) && !a->C) return fail(BSG_ERR_INVALID_PROBLEM, "beta needs the C array");
  int64_t max_n = 0, total_rows = 0;
  for (int g = 0; g < a->num_groups; ++g) {
    const PtrGroup r = ptr_group(a, g);
    if (r.M < 0 || r.N < 0 || r.K < 1) return fail(BSG_ERR_INVALID_PROBLEM, "group %d: extents M=%lld N=%lld K=%lld", g, (long long)r.M, (long long)r.N, (long long)r.K);
    if (r.M == 0 || r.N == 0) continue;
    Problem q;
    memset(&q, 0, sizeof(q));
    q.kind = a->kind; q.out_kind = a->out_kind; q.num_groups = 1;
    q.rows_per_group = r.M; q.total_rows = r.M; q.N = r.N; q.K = r.K;
    q.A = r.A; q.B = r.B; q.SFA = r.SFA; q.SFB = r.SFB; q.C = r.C; q.D = r.D; q.SFD = r.SFD;
    q.b_per_group = true;
    q.lda = r.lda; q.ldb = r.ldb; q.ldc = r.ldc; q.ldd = r.ldd;
    q.alpha = a->alpha; q.beta = r.C ? a->beta : 0.0f; q.norm_ptr = a->norm_constant;
    q.activation = a->activation; q.cta_group = 2;
    Plan plan;
    const int32_t rc = validate(q, &plan);
    if (rc != BSG_OK) {
      char inner[400];
      snprintf(inner, sizeof(inner), "%s", g_err);
      return fail(rc, "group %d: %s", g, inner);
    }
    if ((a->beta != 0.0f || a->beta_array) && !r.C) return fail(BSG_ERR_INVALID_PROBLEM, "group %d: beta needs C", g);
    max_n = r.N > max_n ? r.N : max_n;
    total_rows += r.M;
  }
  const int32_t tn = a->tile_n ? a->tile_n : (max_n > 128 ? 256 : 128);
  int64_t tiles = 0;
  for (int g = 0; g < a->num_groups; ++g) {
    const int64_t M = a->problem_sizes[3 * g], N = a->problem_sizes[3 * g + 1];
    tiles += ((M + 255) / 256) * ((N + tn - 1) / tn);
  }
  if (tiles > 0x3FFFFFFF) return fail(BSG_ERR_INVALID_PROBLEM, "too many tiles for one launch");
  info->kind = a->kind; info->out_kind = a->out_kind; info->num_groups = a->num_groups; info->tile_n = tn;
  info->total_tiles = tiles; info->total_rows = total_rows;
  info->sizes_hash = hash_sizes(a->problem_sizes, 3 * a->num_groups);
  return BSG_OK;
}

template <int KIND, int BN>
int32_t ptr_array_encode(const bsg_ptr_array_args* a, bsg::GroupDesc* table) {
  using Cf = bsg::Cfg<KIND, 2, BN>;
  const bool fp4 = bsg::kind_packs_fp4(KIND);
  for (int g = 0; g < a->num_groups; ++g) {
    const PtrGroup r = ptr_group(a, g);
    bsg::GroupDesc& d = table[g];
    d.M = int32_t(r.M); d.N = int32_t(r.N); d.K = int32_t(r.K);
    d.C = static_cast<const __nv_bfloat16*>(r.C); d.D = r.D; d.SFD = static_cast<uint8_t*>(r.SFD);
    d.ldc = r.ldc; d.ldd = r.ldd;
    if (r.M == 0 || r.N == 0) continue;
    const uint64_t k_bytes = uint64_t(fp4 ? r.K / 2 : r.K);
    const uint64_t lda_bytes = uint64_t(fp4 ? r.lda / 2 : r.lda), ldb_bytes = uint64_t(fp4 ? r.ldb / 2 : r.ldb);
    const uint64_t k_atoms = uint64_t(((r.K + Cf::kSfVec - 1) / Cf::kSfVec + 3) / 4);
    int32_t rc;
    if ((rc = make_operand_map(&d.tmA, r.A, k_bytes, uint64_t(r.M), 1, lda_bytes, uint64_t(r.M) * lda_bytes, Cf::kCtaM)) != BSG_OK) return rc;
    if ((rc = make_operand_map(&d.tmB, r.B, k_bytes, uint64_t(r.N), 1, ldb_bytes, uint64_t(r.N) * ldb_bytes, Cf::kBRowsCta)) != BSG_OK) return rc;
    if ((rc = make_sf_map(&d.tmSFA, r.SFA, k_atoms, uint64_t((r.M + 127) / 128), Cf::kKAtoms, 1)) != BSG_OK) return rc;
    if ((rc = make_sf_map(&d.tmSFB, r.SFB, k_atoms, uint64_t((r.N + 127) / 128), Cf::kKAtoms, Cf::kSfbAtoms)) != BSG_OK) return rc;
    if ((rc = make_out_map(&d.tmD, r.D, a->out_kind, uint64_t(r.N), uint64_t(r.M), 1, uint64_t(r.ldd), uint64_t(r.M) * uint64_t(r.ldd))) != BSG_OK) return rc;
  }
  return BSG_OK;
}

template <int KIND, int BN, bool OUTX>
int32_t ptr_array_launch(const bsg_ptr_array_args* a, const PtrTableInfo& info, uint8_t* workspace, cudaStream_t stream, int sms, int dev) {
  using Cf = bsg::Cfg<KIND, 2, BN>;
  bsg::GemmParams p;
  memset(&p, 0, sizeof(p));
  p.num_groups = a->num_groups;
  p.total_rows = int32_t(info.total_rows);
  p.raster_band = a->raster_band > 0 ? a->raster_band : 16;
  p.out_kind = a->out_kind;
  p.alpha = a->alpha; p.beta = a->beta;
  p.alpha_array = a->alpha_array; p.beta_array = a->beta_array;
  p.norm_ptr = a->norm_constant;
  p.activation = a->activation;
  p.status = reinterpret_cast<uint32_t*>(workspace);
  p.split_tail = 1;
  p.group_desc = reinterpret_cast<const bsg::GroupDesc*>(workspace + kPtrTableOffset);
  int max_clusters = 0;
  int32_t rc = kernel_setup<KIND, 2, BN, false, false, false, true, OUTX>(dev, &max_clusters);
  if (rc != BSG_OK) return rc;
  int64_t clusters = sms / 2;
  if (max_clusters > 0 && clusters > max_clusters) clusters = max_clusters;
  if (info.total_tiles < clusters) clusters = info.total_tiles;
  if (clusters < 1) clusters = 1;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(unsigned(clusters * 2), 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cf::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (a->use_pdl) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  // The six map parameters of the kernel are not used in this form (every group brings its own in the table).
  CUtensorMap none;
  memset(&none, 0, sizeof(none));
  cudaError_t e = cudaLaunchKernelEx(&cfg, bsg::bsg_gemm_kernel<KIND, 2, BN, false, false, false, true, OUTX>, none, none, none, none, none, none, p);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  return BSG_OK;
}

Problem from_dense(const bsg_gemm_args* a) {
  Problem q;
  memset(&q, 0, sizeof(q));
  q.kind = a->kind;
  q.out_kind = a->out_kind;
  q.num_groups = a->batch < 1 ? 1 : a->batch;
  q.rows_per_group = a->M;
  q.total_rows = a->M * q.num_groups;
  q.N = a->N;
  q.K = a->K;
  q.A = a->A; q.B = a->B; q.SFA = a->SFA; q.SFB = a->SFB; q.C = a->C; q.D = a->D; q.SFD = a->SFD;
  q.offsets = nullptr;
  q.b_per_group = true;
  q.ldc = a->ldc ? a->ldc : a->N;
  q.out_col_major = a->out_layout == BSG_LAYOUT_COL_MAJOR ? 1 : 0;
  q.ldd = a->ldd ? a->ldd : (q.out_col_major ? a->M : a->N);
  q.lda = a->lda ? a->lda : a->K;
  q.ldb = a->ldb ? a->ldb : a->K;
  q.bs_a = a->batch_stride_A ? a->batch_stride_A : a->M * q.lda;
  q.bs_b = a->batch_stride_B ? a->batch_stride_B : a->N * q.ldb;
  q.bs_c = a->batch_stride_C ? a->batch_stride_C : a->M * q.ldc;
  q.bs_d = a->batch_stride_D ? a->batch_stride_D : a->M * q.ldd;
  q.use_pdl = a->use_pdl; q.scheduler = a->scheduler;
  q.cluster[0] = a->cluster_m; q.cluster[1] = a->cluster_n; q.cluster[2] = a->cluster_fallback_m; q.cluster[3] = a->cluster_fallback_n;
  q.alpha = a->alpha; q.beta = a->beta;
  q.alpha_ptr = a->alpha_ptr; q.beta_ptr = a->beta_ptr; q.norm_ptr = a->norm_constant;
  q.tile_n = a->tile_n; q.cta_group = a->cta_group; q.sm_count = a->sm_count; q.raster_band = a->raster_band;
  q.bias = a->bias_mode != BSG_BIAS_NONE ? a->bias : nullptr;
  q.bias_mode = a->bias_mode; q.bias_group_stride = 0; q.activation = a->activation;
  return q;
}

Problem from_grouped(const bsg_grouped_args* a) {
  Problem q;
  memset(&q, 0, sizeof(q));
  q.kind = a->kind;
  q.out_kind = a->out_kind;
  q.num_groups = a->num_groups;
  q.rows_per_group = 0;
  q.total_rows = a->total_M;
  q.N = a->N;
  q.K = a->K;
  q.A = a->A; q.B = a->B; q.SFA = a->SFA; q.SFB = a->SFB; q.C = a->C; q.D = a->D; q.SFD = a->SFD;
  q.norm_ptr = a->norm_constant;
  q.offsets = a->offsets;
  q.b_per_group = true;
  q.ldc = a->ldc ? a->ldc : a->N;
  q.ldd = a->ldd ? a->ldd : a->N;
  q.lda = a->K; q.ldb = a->K;
  q.bs_b = a->N * a->K;
  q.use_pdl = a->use_pdl; q.scheduler = a->scheduler;
  q.alpha = a->alpha; q.beta = a->beta;
  q.tile_n = a->tile_n; q.cta_group = a->cta_group; q.sm_count = a->sm_count; q.raster_band = a->raster_band;
  q.bias = a->bias; q.bias_mode = a->bias ? BSG_BIAS_PER_COLUMN : BSG_BIAS_NONE; q.bias_group_stride = int32_t(a->N);
  q.activation = a->activation;
  q.alpha_array = a->alpha_array; q.beta_array = a->beta_array;
  return q;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Scratch for bsg_gemm_run_static: the kernel's workspace (today a 16-byte status word) lives in
// this fixed device array instead of caller-provided memory.  Every GPU that loads the library
// holds these 256 bytes until the process exits.  In host code the name below is only a stand-in
// for the symbol; the device address is looked up once per device with cudaGetSymbolAddress.
constexpr size_t kStaticScratchBytes = 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Device address of g_static_scratch on the current device (resolved on first use, then cached).
int32_t static_scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(BSG_ERR_NOT_SUPPORTED, "device ordinal %d is outside [0, %d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) return fail(BSG_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return BSG_OK;
}
}  // namespace

// Per-rank state of the tensor-parallel GEMM: one device allocation that holds the full-size A and
// SFA buffers (this rank's shard in place, the others filled in by the kernel) and the sync words.
struct bsg_tp_comm {
  int32_t rank, world, kind;
  int64_t M, K, rows_per_shard;
  int64_t row_bytes, k_atoms, sfa_rowatom_bytes;
  size_t a_off, sfa_off, sync_off, total_bytes;
  size_t a_bytes, sfa_bytes;   // one gathered buffer each; two of each lie back to back
  uint8_t* base;
  uint8_t* peer_base[8];
  bool opened[8];
  bool connected;
  uint32_t epoch;
  int32_t mode;            // BSG_TP_PUSH_KERNEL / BSG_TP_PUSH_COPY_ENGINE
  cudaStream_t side;       // set-up work; copy-engine mode: first of the transfer streams
  cudaStream_t lanes[4];   // copy-engine mode: parallel transfer streams (lanes[0] == side)
  cudaEvent_t ev_start, ev_done, ev_lane[4];
};

// Per-rank state of the GEMM + reduce-scatter: one device allocation with the receive buffers (two halves used by
// alternate calls, world - 1 slices of M / world x N bf16 each), the arrival counters of their tiles, and the sync words.
struct bsg_rs_comm {
  int32_t rank, world, flags;
  int64_t M, N, slice_rows, tiles_per_slice, tiles_n;
  size_t recv_off, flags_off, sync_off, maps_off, out_off, total_bytes;   // out: two halves of M x N bf16 (all-reduce only)
  uint8_t* base;
  uint8_t* peer_base[8];
  bool opened[8];
  bool connected;
  uint32_t epoch;
  uint32_t ar_calls;      // all-reduce calls so far (the arrival counter counts only those)
  bool maps_uploaded;
};

// All-reduce: one map per rank over its output (N columns, M rows, two halves), stored in this rank's own memory where
// the kernel reads them.
static int32_t rs_upload_out_maps(bsg_rs_comm* c) {
  CUtensorMap maps[8];
  memset(maps, 0, sizeof(maps));
  for (int q = 0; q < c->world; ++q) {
    const int32_t rc = make_out_map(&maps[q], c->peer_base[q] + c->out_off, BSG_OUT_BF16, uint64_t(c->N), uint64_t(c->M), 2, uint64_t(c->N),
                                    uint64_t(c->M) * uint64_t(c->N));
    if (rc != BSG_OK) return rc;
  }
  cudaError_t e = cudaMemcpy(c->base + c->maps_off, maps, sizeof(maps), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "uploading the output maps: %s", cudaGetErrorString(e));
  c->maps_uploaded = true;
  return BSG_OK;
}

extern "C" {

int32_t bsg_version(void) { return 100; }

const char* bsg_last_error_string(void) { return g_err; }

int32_t bsg_gemm_query(const bsg_gemm_args* args, bsg_caps* caps) {
  if (!args) return fail(BSG_ERR_INVALID_PROBLEM, "args is null");
  if (args->M < 0 || args->batch < 0) return fail(BSG_ERR_INVALID_PROBLEM, "negative extent");
  Problem q = from_dense(args);
  Plan plan;
  int32_t rc = validate(q, &plan);
  if (rc != BSG_OK) return rc;
  fill_caps(q, plan, caps);
  return BSG_OK;
}

int32_t bsg_grouped_query(const bsg_grouped_args* args, bsg_caps* caps) {
  if (!args) return fail(BSG_ERR_INVALID_PROBLEM, "args is null");
  if (!args->offsets) return fail(BSG_ERR_INVALID_PROBLEM, "offsets is null");
  Problem q = from_grouped(args);
  Plan plan;
  int32_t rc = validate(q, &plan);
  if (rc != BSG_OK) return rc;
  fill_caps(q, plan, caps);
  return BSG_OK;
}

int32_t bsg_gemm_workspace_size(const bsg_gemm_args* args, size_t* bytes) {
  if (!args || !bytes) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  *bytes = 16;
  return BSG_OK;
}

int32_t bsg_grouped_workspace_size(const bsg_grouped_args* args, size_t* bytes) {
  if (!args || !bytes) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  *bytes = 16;
  return BSG_OK;
}

int32_t bsg_gemm_run(const bsg_gemm_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (!args) return fail(BSG_ERR_INVALID_PROBLEM, "args is null");
  if (args->M < 0 || args->batch < 0) return fail(BSG_ERR_INVALID_PROBLEM, "negative extent");
  Problem q = from_dense(args);
  return run_problem(q, workspace, workspace_bytes, cuda_stream);
}

int32_t bsg_grouped_run(const bsg_grouped_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (!args) return fail(BSG_ERR_INVALID_PROBLEM, "args is null");
  if (!args->offsets) return fail(BSG_ERR_INVALID_PROBLEM, "offsets is null");
  Problem q = from_grouped(args);
  return run_problem(q, workspace, workspace_bytes, cuda_stream);
}

int32_t bsg_workspace_init(void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (!workspace) return fail(BSG_ERR_WORKSPACE_NULL, "workspace is null");
  if (workspace_bytes < 16) return fail(BSG_ERR_WORKSPACE_NULL, "workspace smaller than 16 bytes");
  cudaError_t e = cudaMemsetAsync(workspace, 0, 16, static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  return BSG_OK;
}

int32_t bsg_read_device_status(void* workspace, void* cuda_stream) {
  if (!workspace) return fail(BSG_ERR_WORKSPACE_NULL, "workspace is null");
  uint32_t st = 0;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaMemcpyAsync(&st, workspace, sizeof(st), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "reading status: %s", cudaGetErrorString(e));
  if (st == 0) return BSG_OK;
  e = cudaMemsetAsync(workspace, 0, 16, stream);   // the status is sticky until it has been read
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "clearing status: %s", cudaGetErrorString(e));
  if (st & bsg::kStBadOffsets) return fail(BSG_ERR_INVALID_PROBLEM, "group offsets are not monotone or exceed total_M (device status 0x%x)", st);
  return fail(BSG_ERR_TIMEOUT, "a bounded device-side wait ran out (device status 0x%x)", st);
}

int32_t bsg_gemm_run_static(const bsg_gemm_args* args, void* cuda_stream, uint32_t* device_status_out) {
  if (!args) return fail(BSG_ERR_INVALID_PROBLEM, "args is null");
  if (args->M < 0 || args->batch < 0) return fail(BSG_ERR_INVALID_PROBLEM, "negative extent");
  // Arguments are checked first: a refused call puts nothing on the stream and leaves the shared array alone.
  Problem q = from_dense(args);
  Plan plan;
  int32_t rc = validate(q, &plan);
  if (rc != BSG_OK) return rc;
  size_t need = 0;
  rc = bsg_gemm_workspace_size(args, &need);
  if (rc != BSG_OK) return rc;
  if (need > kStaticScratchBytes)
    return fail(BSG_ERR_NOT_SUPPORTED, "this problem needs %zu bytes of scratch but the built-in scratch holds %zu; use bsg_gemm_run with a caller-provided workspace",
                need, kStaticScratchBytes);
  void* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);
  if (rc != BSG_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // The array still holds what the previous call left there: the status word must start at zero.
  cudaError_t e = cudaMemsetAsync(scratch, 0, need, stream);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "clearing the static scratch: %s", cudaGetErrorString(e));
  rc = run_problem(q, scratch, kStaticScratchBytes, cuda_stream);
  if (rc != BSG_OK) return rc;
  if (device_status_out) {
    uint32_t st = 0;
    e = cudaMemcpyAsync(&st, scratch, sizeof(st), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "reading the static scratch: %s", cudaGetErrorString(e));
    *device_status_out = st;
    // Same translation as bsg_read_device_status: the raw word goes to the caller, the meaning into the return code.
    if (st != 0) return fail(BSG_ERR_TIMEOUT, "a bounded device-side wait ran out (device status 0x%x)", st);
  }
  return BSG_OK;
}

int32_t bsg_quantize(const bsg_quant_args* a, void* cuda_stream) {
  if (!a) return fail(BSG_ERR_INVALID_PROBLEM, "args is null");
  if (a->kind != BSG_KIND_NVFP4 && a->kind != BSG_KIND_MXFP8) return fail(BSG_ERR_NOT_SUPPORTED, "unknown operand kind %d", a->kind);
  if (a->rows < 0 || a->K < 1) return fail(BSG_ERR_INVALID_PROBLEM, "extents must be positive (rows=%lld K=%lld)", (long long)a->rows, (long long)a->K);
  if (a->rows > int64_t(65535) * bsg::kQuantTileRows || a->K > 0x3FFFFFFF) return fail(BSG_ERR_INVALID_PROBLEM, "extent too large");
  if (a->K % 32 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "K=%lld must be a multiple of 32", (long long)a->K);
  if (a->ldx < a->K || a->ldx % 8 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "ldx=%lld must be >= K and a multiple of 8 elements", (long long)a->ldx);
  if (a->rows == 0) return BSG_OK;
  if (!a->X || !a->Q || !a->SF) return fail(BSG_ERR_INVALID_PROBLEM, "X, Q and SF must not be null");
  if (!aligned16(a->X) || !aligned16(a->Q) || !aligned16(a->SF)) return fail(BSG_ERR_MISALIGNED_OPERAND, "X, Q and SF must be 16-byte aligned");
  const int64_t vec = a->kind == BSG_KIND_NVFP4 ? 16 : 32;
  bsg::QuantParams p{};
  p.X = static_cast<const uint16_t*>(a->X); p.Q = static_cast<uint8_t*>(a->Q); p.SF = static_cast<uint8_t*>(a->SF);
  p.norm_ptr = a->norm_constant; p.ldx = a->ldx; p.rows = int32_t(a->rows); p.K = int32_t(a->K);
  p.k_atoms = int32_t((a->K / vec + 3) / 4);
  dim3 grid(unsigned((a->K + bsg::kQuantTileK - 1) / bsg::kQuantTileK), unsigned((a->rows + bsg::kQuantTileRows - 1) / bsg::kQuantTileRows));
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (a->use_pdl != 0 && a->use_pdl != 1) return fail(BSG_ERR_INVALID_PROBLEM, "use_pdl must be 0 or 1");
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = dim3(bsg::kQuantThreads, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a->use_pdl ? 1 : 0;
  cudaError_t e = a->kind == BSG_KIND_NVFP4 ? cudaLaunchKernelEx(&cfg, bsg::bsg_quant_kernel<0>, p) : cudaLaunchKernelEx(&cfg, bsg::bsg_quant_kernel<1>, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "quantiser launch: %s", cudaGetErrorString(e));
  return BSG_OK;
}

int32_t bsg_ptr_array_workspace_size(const bsg_ptr_array_args* args, size_t* bytes) {
  if (!args || !bytes) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  if (args->num_groups < 1 || args->num_groups > BSG_MAX_GROUPS) return fail(BSG_ERR_INVALID_PROBLEM, "group count %d outside [1, %d]", args->num_groups, BSG_MAX_GROUPS);
  *bytes = kPtrTableOffset + size_t(args->num_groups) * sizeof(bsg::GroupDesc);
  return BSG_OK;
}

int32_t bsg_ptr_array_initialize(const bsg_ptr_array_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  PtrTableInfo info;
  int32_t rc = ptr_array_check(args, &info);
  if (rc != BSG_OK) return rc;
  if (!workspace) return fail(BSG_ERR_WORKSPACE_NULL, "workspace is null");
  const size_t need = kPtrTableOffset + size_t(args->num_groups) * sizeof(bsg::GroupDesc);
  if (workspace_bytes < need) return fail(BSG_ERR_WORKSPACE_NULL, "workspace of %zu bytes is smaller than the %zu needed", workspace_bytes, need);
  if ((reinterpret_cast<uintptr_t>(workspace) & 127u) != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "the workspace of the pointer-array form must be 128-byte aligned");
  bsg::GroupDesc* table = static_cast<bsg::GroupDesc*>(calloc(size_t(args->num_groups), sizeof(bsg::GroupDesc)));
  if (!table) return fail(BSG_ERR_INTERNAL, "out of host memory");
  g_bypass_map_cache = true;
  if (args->kind == BSG_KIND_NVFP4) rc = info.tile_n == 256 ? ptr_array_encode<0, 256>(args, table) : ptr_array_encode<0, 128>(args, table);
  else rc = info.tile_n == 256 ? ptr_array_encode<1, 256>(args, table) : ptr_array_encode<1, 128>(args, table);
  g_bypass_map_cache = false;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaSuccess;
  if (rc == BSG_OK) {
    e = cudaMemsetAsync(workspace, 0, 16, stream);
    // pageable source: the copy has left the host buffer when the call returns
    if (e == cudaSuccess) e = cudaMemcpyAsync(static_cast<uint8_t*>(workspace) + kPtrTableOffset, table, size_t(args->num_groups) * sizeof(bsg::GroupDesc), cudaMemcpyHostToDevice, stream);
  }
  free(table);
  if (rc != BSG_OK) return rc;
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "uploading the group table: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(g_ptr_tables_mutex);
  int slot = -1;
  for (int i = 0; i < kPtrTables; ++i) if (g_ptr_tables[i].ws == workspace) { slot = i; break; }
  if (slot < 0) { slot = g_ptr_tables_next; g_ptr_tables_next = (g_ptr_tables_next + 1) % kPtrTables; }
  g_ptr_tables[slot].ws = workspace;
  g_ptr_tables[slot].info = info;
  return BSG_OK;
}

int32_t bsg_ptr_array_initialize_from_device(const bsg_ptr_array_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (!args) return fail(BSG_ERR_INVALID_PROBLEM, "args is null");
  if (args->num_groups < 1 || args->num_groups > BSG_MAX_GROUPS) return fail(BSG_ERR_INVALID_PROBLEM, "group count %d outside [1, %d]", args->num_groups, BSG_MAX_GROUPS);
  const size_t n = size_t(args->num_groups);
  // host copies of the twelve arrays: sizes (3 int32 per group), seven pointer arrays, four pitch arrays
  int32_t sizes[3 * BSG_MAX_GROUPS];
  static_assert(sizeof(void*) == sizeof(int64_t), "pointer and pitch arrays share the staging type");
  int64_t* host = static_cast<int64_t*>(malloc(11 * n * sizeof(int64_t)));
  if (!host) return fail(BSG_ERR_INTERNAL, "out of host memory");
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  bsg_ptr_array_args local = *args;
  cudaError_t e = cudaSuccess;
  auto fetch = [&](const void* dev_array, void* dst, size_t bytes) {
    if (dev_array && e == cudaSuccess) e = cudaMemcpyAsync(dst, dev_array, bytes, cudaMemcpyDeviceToHost, stream);
  };
  fetch(args->problem_sizes, sizes, 3 * n * sizeof(int32_t));
  const void* const dev_arrays[11] = {args->A, args->B, args->SFA, args->SFB, args->C, args->D, args->SFD, args->lda, args->ldb, args->ldc, args->ldd};
  for (int i = 0; i < 11; ++i) fetch(dev_arrays[i], host + size_t(i) * n, n * sizeof(int64_t));
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) { free(host); return fail(BSG_ERR_CUDA, "copying the argument arrays to the host: %s", cudaGetErrorString(e)); }
  auto at = [&](int i) { return dev_arrays[i] ? host + size_t(i) * n : nullptr; };
  local.problem_sizes = args->problem_sizes ? sizes : nullptr;
  local.A = reinterpret_cast<const void* const*>(at(0)); local.B = reinterpret_cast<const void* const*>(at(1));
  local.SFA = reinterpret_cast<const void* const*>(at(2)); local.SFB = reinterpret_cast<const void* const*>(at(3));
  local.C = reinterpret_cast<const void* const*>(at(4));
  local.D = reinterpret_cast<void* const*>(at(5)); local.SFD = reinterpret_cast<void* const*>(at(6));
  local.lda = at(7); local.ldb = at(8); local.ldc = at(9); local.ldd = at(10);
  const int32_t rc = bsg_ptr_array_initialize(&local, workspace, workspace_bytes, cuda_stream);
  free(host);
  return rc;
}

int32_t bsg_ptr_array_run(const bsg_ptr_array_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (!args || !args->problem_sizes) return fail(BSG_ERR_INVALID_PROBLEM, "args or problem_sizes is null");
  if (!workspace) return fail(BSG_ERR_WORKSPACE_NULL, "workspace is null");
  if (args->num_groups < 1 || args->num_groups > BSG_MAX_GROUPS) return fail(BSG_ERR_INVALID_PROBLEM, "group count %d outside [1, %d]", args->num_groups, BSG_MAX_GROUPS);
  PtrTableInfo info;
  {
    std::lock_guard<std::mutex> lock(g_ptr_tables_mutex);
    int slot = -1;
    for (int i = 0; i < kPtrTables; ++i) if (g_ptr_tables[i].ws == workspace) { slot = i; break; }
    if (slot < 0) return fail(BSG_ERR_INVALID_PROBLEM, "bsg_ptr_array_initialize has not been called for this workspace");
    info = g_ptr_tables[slot].info;
  }
  if (info.kind != args->kind || info.out_kind != args->out_kind || info.num_groups != args->num_groups ||
      info.sizes_hash != hash_sizes(args->problem_sizes, 3 * args->num_groups) || (args->tile_n != 0 && args->tile_n != info.tile_n))
    return fail(BSG_ERR_INVALID_PROBLEM, "the arguments differ from those the workspace was initialised with");
  if (workspace_bytes < kPtrTableOffset + size_t(args->num_groups) * sizeof(bsg::GroupDesc)) return fail(BSG_ERR_WORKSPACE_NULL, "workspace too small");
  if (args->use_pdl != 0 && args->use_pdl != 1) return fail(BSG_ERR_INVALID_PROBLEM, "use_pdl must be 0 or 1");
  if (args->activation < BSG_ACT_IDENTITY || args->activation > BSG_ACT_SILU) return fail(BSG_ERR_NOT_SUPPORTED, "unknown activation %d", args->activation);
  if (args->out_kind == BSG_OUT_NVFP4 && !args->norm_constant) return fail(BSG_ERR_INVALID_PROBLEM, "NVFP4 output needs norm_constant");
  if ((args->beta != 0.0f || args->beta_array) && !args->C) return fail(BSG_ERR_INVALID_PROBLEM, "beta needs the C array");
  int dev = 0, major = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (major != 10) return fail(BSG_ERR_ARCH_MISMATCH, "device compute capability %d.x is not sm_100", major);
  if (args->sm_count > 0 && args->sm_count < sms) sms = args->sm_count;
  if (info.total_tiles == 0) return BSG_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const bool outx = args->out_kind >= BSG_OUT_F16;
  if (args->kind == BSG_KIND_NVFP4) {
    if (outx) return info.tile_n == 256 ? ptr_array_launch<0, 256, true>(args, info, ws, stream, sms, dev) : ptr_array_launch<0, 128, true>(args, info, ws, stream, sms, dev);
    return info.tile_n == 256 ? ptr_array_launch<0, 256, false>(args, info, ws, stream, sms, dev) : ptr_array_launch<0, 128, false>(args, info, ws, stream, sms, dev);
  }
  if (outx) return info.tile_n == 256 ? ptr_array_launch<1, 256, true>(args, info, ws, stream, sms, dev) : ptr_array_launch<1, 128, true>(args, info, ws, stream, sms, dev);
  return info.tile_n == 256 ? ptr_array_launch<1, 256, false>(args, info, ws, stream, sms, dev) : ptr_array_launch<1, 128, false>(args, info, ws, stream, sms, dev);
}

int32_t bsg_tp_create(int32_t rank, int32_t world, int32_t kind, int64_t M, int64_t K, bsg_tp_comm** out, void* ipc_handle_out) {
  if (!out || !ipc_handle_out) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(BSG_ERR_INVALID_PROBLEM, "rank %d / world %d outside [0, 8]", rank, world);
  if (kind != BSG_KIND_NVFP4 && kind != BSG_KIND_MXFP8) return fail(BSG_ERR_NOT_SUPPORTED, "unknown operand kind %d", kind);
  if (M < 1 || K < 1 || M % (int64_t(world) * 256) != 0) return fail(BSG_ERR_INVALID_PROBLEM, "M=%lld must be a multiple of 256 * world", (long long)M);
  const int64_t vec = kind == BSG_KIND_NVFP4 ? 16 : 32;
  const int64_t row_bytes = kind == BSG_KIND_NVFP4 ? K / 2 : K;
  if (K % (kind == BSG_KIND_NVFP4 ? 32 : 16) != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "K=%lld is not 16-byte aligned per row", (long long)K);
  bsg_tp_comm* c = new (std::nothrow) bsg_tp_comm();
  if (!c) return fail(BSG_ERR_INTERNAL, "out of host memory");
  memset(c, 0, sizeof(*c));
  c->rank = rank; c->world = world; c->kind = kind; c->M = M; c->K = K; c->rows_per_shard = M / world;
  c->row_bytes = row_bytes;
  c->k_atoms = ((K + vec - 1) / vec + 3) / 4;
  c->sfa_rowatom_bytes = 512 * c->k_atoms;
  const size_t a_bytes = size_t(M) * size_t(row_bytes);
  const size_t sfa_bytes = size_t(M / 128) * size_t(c->sfa_rowatom_bytes);
  const size_t sync_bytes = (size_t(bsg::kTpSyncFlags) + size_t(M / 256)) * 4;
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  // Two gathered buffers of each kind, back to back: call n fills and reads buffer n & 1, so a peer may
  // already push the data of the next call while this rank still computes on the current one.  This
  // rank's own rows always stay in buffer 0 (where the caller writes them).
  c->a_bytes = a_bytes; c->sfa_bytes = sfa_bytes;
  c->a_off = 0;
  c->sfa_off = up(2 * a_bytes);
  c->sync_off = c->sfa_off + up(2 * sfa_bytes);
  c->total_bytes = c->sync_off + up(sync_bytes);
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->base), c->total_bytes);
  if (e != cudaSuccess) { delete c; return fail(BSG_ERR_CUDA, "cudaMalloc(%zu): %s", c->total_bytes, cudaGetErrorString(e)); }
  e = cudaMemset(c->base + c->sync_off, 0, up(sync_bytes));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, c->base);
  if (e != cudaSuccess) { cudaFree(c->base); delete c; return fail(BSG_ERR_CUDA, "tensor-parallel buffer set-up: %s", cudaGetErrorString(e)); }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(ipc_handle_out, &h, 64);
  c->peer_base[rank] = c->base;
  // Spread push: on 4 GPUs 8 % faster than the eager push and 2 % faster than the paced one.  Release-fenced announcements:
  // with relaxed ones, eight ranks running 50 small calls in a row (2048 rows, 128 columns per rank, K 1024) had one rank
  // read a row block before its rows had landed; the counter had overtaken the data.
  c->mode = BSG_TP_PUSH_KERNEL | BSG_TP_SPREAD_PUSH | BSG_TP_RELEASE_ANNOUNCE;
  e = cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_start, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_done, cudaEventDisableTiming);
  c->lanes[0] = c->side;
  for (int i = 0; i < 4 && e == cudaSuccess; ++i) {
    if (i > 0) e = cudaStreamCreateWithFlags(&c->lanes[i], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_lane[i], cudaEventDisableTiming);
  }
  if (e != cudaSuccess) { cudaFree(c->base); delete c; return fail(BSG_ERR_CUDA, "tensor-parallel stream set-up: %s", cudaGetErrorString(e)); }
  c->connected = world == 1;
  *out = c;
  return BSG_OK;
}

int32_t bsg_tp_connect(bsg_tp_comm* c, const void* all_handles) {
  if (!c || !all_handles) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  for (int q = 0; q < c->world; ++q) {
    if (q == c->rank || c->opened[q]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(all_handles) + size_t(q) * 64, 64);
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", q, cudaGetErrorString(e));
    c->peer_base[q] = static_cast<uint8_t*>(ptr);
    c->opened[q] = true;
  }
  // First use of a kernel or of a peer mapping can need work in the driver that does not overlap a running
  // persistent GEMM: do it now, once, on the side stream (unused sync words 16..31 serve as targets).
  uint32_t* own_sync = reinterpret_cast<uint32_t*>(c->base + c->sync_off);
  bsg::tp_wait_peers_kernel<<<1, 32, 0, c->side>>>(own_sync, 1, 0, 0, nullptr);
  bsg::tp_announce_kernel<<<1, 32, 0, c->side>>>(own_sync + 16, 0, 0, 0);
  cudaError_t e = cudaGetLastError();
  for (int q = 0; q < c->world && e == cudaSuccess; ++q) {
    if (q == c->rank) continue;
    e = cudaMemcpyAsync(c->peer_base[q] + c->sync_off + size_t(16 + c->rank) * 4, own_sync + 31, 4, cudaMemcpyDeviceToDevice, c->side);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->side);
  if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "tensor-parallel warm-up: %s", cudaGetErrorString(e));
  c->connected = true;
  return BSG_OK;
}

int32_t bsg_tp_buffers(bsg_tp_comm* c, void** a_full, void** sfa_full, void** a_shard, void** sfa_shard) {
  if (!c) return fail(BSG_ERR_INVALID_PROBLEM, "null communicator");
  uint8_t* a = c->base + c->a_off;
  uint8_t* sf = c->base + c->sfa_off;
  if (a_full) *a_full = a;
  if (sfa_full) *sfa_full = sf;
  if (a_shard) *a_shard = a + size_t(c->rank) * size_t(c->rows_per_shard) * size_t(c->row_bytes);
  if (sfa_shard) *sfa_shard = sf + size_t(c->rank) * size_t(c->rows_per_shard / 128) * size_t(c->sfa_rowatom_bytes);
  return BSG_OK;
}

int32_t bsg_tp_gemm_run(bsg_tp_comm* c, const bsg_gemm_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (!c || !args) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  if (!c->connected) return fail(BSG_ERR_INVALID_PROBLEM, "bsg_tp_connect has not been called");
  if (args->M != c->M || args->K != c->K || args->kind != c->kind) return fail(BSG_ERR_INVALID_PROBLEM, "M, K and kind must match the communicator");
  if (args->batch > 1) return fail(BSG_ERR_NOT_SUPPORTED, "the tensor-parallel GEMM is not batched");
  bsg_gemm_args local = *args;
  local.batch = 1;
  local.A = c->base + c->a_off;
  local.SFA = c->base + c->sfa_off;
  local.cta_group = 2;
  Problem q = from_dense(&local);
  q.tp = true;
  q.tp_world = c->world; q.tp_rank = c->rank; q.tp_rows_per_shard = int32_t(c->rows_per_shard);
  int ks = 32;   // pieces per 256-row block: A by rows (256 / ks each), SFA by k-atoms
  while (ks > 1 && c->k_atoms % ks != 0) ks >>= 1;
  q.tp_ksplit = ks;
  q.tp_row_bytes = c->row_bytes; q.tp_sfa_rowatom_bytes = c->sfa_rowatom_bytes;
  q.tp_epoch = c->epoch + 1;
  const bool single_buffer = (c->mode & BSG_TP_SINGLE_BUFFER) != 0;
  q.tp_parity = single_buffer ? 0 : int32_t(q.tp_epoch & 1u);
  // The buffer this call fills was last read by the peer's previous call (single buffer) or the one before.
  q.tp_ready_target = single_buffer ? q.tp_epoch : q.tp_epoch - 1;
  for (int i = 0; i < c->world; ++i) {
    const bool remote = i != c->rank;     // own entry: the source of the push, always buffer 0
    q.tp_peer_a[i] = c->peer_base[i] + c->a_off + (remote && q.tp_parity ? c->a_bytes : 0);
    q.tp_peer_sfa[i] = c->peer_base[i] + c->sfa_off + (remote && q.tp_parity ? c->sfa_bytes : 0);
    q.tp_peer_sync[i] = reinterpret_cast<uint32_t*>(c->peer_base[i] + c->sync_off);
  }
  // The M sweep starts at this rank's own rows and follows the order in which the shards arrive.
  const int32_t blocks = int32_t(c->rows_per_shard / 256);
  int32_t band = 8;
  while (blocks % band != 0) band >>= 1;
  q.raster_band = band;
  q.tile_m_rotate = c->rank * blocks;
  q.ready_flags = c->world > 1 ? q.tp_peer_sync[c->rank] + bsg::kTpSyncFlags : nullptr;
  q.rows_per_flag = 256;
  q.flag_target = q.tp_epoch * uint32_t(ks);
  const bool copy_engine = c->world > 1 && (c->mode & BSG_TP_PUSH_COPY_ENGINE) != 0;
  q.tp_push_in_kernel = copy_engine ? 0 : 1;
  q.tp_release_announce = (c->mode & BSG_TP_RELEASE_ANNOUNCE) ? 1 : 0;
  q.tp_paced_push = (c->mode & BSG_TP_SPREAD_PUSH) ? 2 : (c->mode & BSG_TP_PACED_PUSH) ? 1 : 0;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (copy_engine) {
    if (!workspace || workspace_bytes < 16) return fail(BSG_ERR_WORKSPACE_NULL, "workspace is null or smaller than 16 bytes");
    // Side stream: once everything enqueued so far on the caller's stream is done (the shard is final)
    // and every peer has launched this call, push the shard to the peers, nearest consumer first, one
    // band of row blocks per transfer, each followed by its announcement.
    cudaError_t e = cudaEventRecord(c->ev_start, stream);
    if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "tensor-parallel stream fork: %s", cudaGetErrorString(e));
  }
  int32_t rc = run_problem(q, workspace, workspace_bytes, cuda_stream);
  if (rc != BSG_OK) return rc;
  if (copy_engine) {
    // A band of row blocks can be cut into slices that travel on parallel streams; measured on two GPUs,
    // four streams made the host-side enqueue the bottleneck (12 operations per band), so one is used.
    uint32_t* own_sync = q.tp_peer_sync[c->rank];
    const int n_lanes = 1;
    const int32_t slice = band / n_lanes;                     // row blocks per transfer
    const int64_t first_block = int64_t(c->rank) * blocks;
    cudaError_t e = cudaSuccess;
    for (int l = 0; l < n_lanes && e == cudaSuccess; ++l) {
      cudaStream_t ls = c->lanes[l];
      e = cudaStreamWaitEvent(ls, c->ev_start, 0);
      if (e != cudaSuccess) break;
      bsg::tp_wait_peers_kernel<<<1, 32, 0, ls>>>(own_sync, c->world, c->rank, q.tp_ready_target, static_cast<uint32_t*>(workspace));
      for (int j = 1; j < c->world && e == cudaSuccess; ++j) {
        const int dst = (c->rank - j + c->world) % c->world;
        for (int32_t b0 = l * slice; b0 < blocks && e == cudaSuccess; b0 += band) {
          const size_t a_off = c->a_off + size_t(first_block + b0) * 256 * size_t(c->row_bytes);
          const size_t a_bytes = size_t(slice) * 256 * size_t(c->row_bytes);
          const size_t s_off = c->sfa_off + size_t(first_block + b0) * 2 * size_t(c->sfa_rowatom_bytes);
          const size_t s_bytes = size_t(slice) * 2 * size_t(c->sfa_rowatom_bytes);
          const size_t a_par = q.tp_parity ? c->a_bytes : 0, s_par = q.tp_parity ? c->sfa_bytes : 0;
          e = cudaMemcpyAsync(c->peer_base[dst] + a_off + a_par, c->base + a_off, a_bytes, cudaMemcpyDeviceToDevice, ls);
          if (e == cudaSuccess) e = cudaMemcpyAsync(c->peer_base[dst] + s_off + s_par, c->base + s_off, s_bytes, cudaMemcpyDeviceToDevice, ls);
          if (e != cudaSuccess) break;
          bsg::tp_announce_kernel<<<1, 32, 0, ls>>>(q.tp_peer_sync[dst] + bsg::kTpSyncFlags, int(first_block + b0), slice, uint32_t(ks));
        }
      }
      // The call is complete on the caller's stream only when the transfers are: the shard may then be rewritten.
      if (e == cudaSuccess) e = cudaGetLastError();
      if (e == cudaSuccess) e = cudaEventRecord(c->ev_lane[l], ls);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(stream, c->ev_lane[l], 0);
    }
    if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "tensor-parallel peer transfers: %s", cudaGetErrorString(e));
  }
  c->epoch += 1;
  return BSG_OK;
}

int32_t bsg_rs_create(int32_t rank, int32_t world, int64_t M, int64_t N, int32_t flags, bsg_rs_comm** out, void* ipc_handle_out) {
  if (!out || !ipc_handle_out) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  if (flags & ~BSG_RS_WITH_ALLREDUCE) return fail(BSG_ERR_NOT_SUPPORTED, "unknown flags 0x%x", flags);
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(BSG_ERR_INVALID_PROBLEM, "rank %d / world %d outside [0, 8]", rank, world);
  if (M < 1 || N < 8 || M % (int64_t(world) * 256) != 0) return fail(BSG_ERR_INVALID_PROBLEM, "M=%lld must be a multiple of 256 * world", (long long)M);
  if (N % 8 != 0) return fail(BSG_ERR_MISALIGNED_OPERAND, "N=%lld must be a multiple of 8", (long long)N);
  bsg_rs_comm* c = new (std::nothrow) bsg_rs_comm();
  if (!c) return fail(BSG_ERR_INTERNAL, "out of host memory");
  memset(c, 0, sizeof(*c));
  c->rank = rank; c->world = world; c->M = M; c->N = N; c->flags = flags;
  c->slice_rows = M / world;
  c->tiles_per_slice = c->slice_rows / 256;
  c->tiles_n = (N + 255) / 256;
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  const size_t stages = size_t(world > 1 ? world - 1 : 1);
  const size_t recv_bytes = 2 * stages * size_t(c->slice_rows) * size_t(N) * 2;
  const size_t flag_bytes = 2 * stages * size_t(c->tiles_per_slice) * size_t(c->tiles_n) * 4;
  c->recv_off = 0;
  c->flags_off = up(recv_bytes);
  c->sync_off = c->flags_off + up(flag_bytes);
  c->maps_off = c->sync_off + 1024;
  c->out_off = c->maps_off + 1024;                 // 8 tensor maps of 128 bytes
  c->total_bytes = c->out_off + ((flags & BSG_RS_WITH_ALLREDUCE) ? 2 * size_t(M) * size_t(N) * 2 : 0);
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->base), c->total_bytes);
  if (e != cudaSuccess) { delete c; return fail(BSG_ERR_CUDA, "cudaMalloc(%zu): %s", c->total_bytes, cudaGetErrorString(e)); }
  e = cudaMemset(c->base + c->flags_off, 0, c->out_off - c->flags_off);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, c->base);
  if (e != cudaSuccess) { cudaFree(c->base); delete c; return fail(BSG_ERR_CUDA, "reduce-scatter buffer set-up: %s", cudaGetErrorString(e)); }
  memcpy(ipc_handle_out, &h, 64);
  c->peer_base[rank] = c->base;
  c->connected = world == 1;
  if (world == 1 && (flags & BSG_RS_WITH_ALLREDUCE)) {      // nobody to connect to: the only output map is this rank's own
    const int32_t rc = rs_upload_out_maps(c);
    if (rc != BSG_OK) { cudaFree(c->base); delete c; return rc; }
  }
  *out = c;
  return BSG_OK;
}

int32_t bsg_rs_connect(bsg_rs_comm* c, const void* all_handles) {
  if (!c || !all_handles) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  // the ring needs the two neighbours only; the all-reduce stores into every rank's output
  const int left_rank = (c->rank + c->world - 1) % c->world, right_rank = (c->rank + 1) % c->world;
  for (int q = 0; q < c->world; ++q) {
    if (!(c->flags & BSG_RS_WITH_ALLREDUCE) && q != left_rank && q != right_rank) continue;
    if (q == c->rank || c->opened[q]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(all_handles) + size_t(q) * 64, 64);
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(BSG_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", q, cudaGetErrorString(e));
    c->peer_base[q] = static_cast<uint8_t*>(ptr);
    c->opened[q] = true;
  }
  if (c->flags & BSG_RS_WITH_ALLREDUCE) {
    const int32_t rc = rs_upload_out_maps(c);
    if (rc != BSG_OK) return rc;
  }
  c->connected = true;
  return BSG_OK;
}

static int32_t rs_run(bsg_rs_comm* c, const bsg_gemm_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream, bool allreduce, void** result) {
  if (!c || !args) return fail(BSG_ERR_INVALID_PROBLEM, "null argument");
  if (!c->connected) return fail(BSG_ERR_INVALID_PROBLEM, "bsg_rs_connect has not been called");
  if (allreduce && !(c->flags & BSG_RS_WITH_ALLREDUCE)) return fail(BSG_ERR_INVALID_PROBLEM, "the communicator was created without BSG_RS_WITH_ALLREDUCE");
  if (allreduce && !c->maps_uploaded) return fail(BSG_ERR_INTERNAL, "the output maps of the all-reduce have not been set up");
  if (args->M != c->M || args->N != c->N) return fail(BSG_ERR_INVALID_PROBLEM, "M and N must match the communicator");
  if (args->batch > 1) return fail(BSG_ERR_NOT_SUPPORTED, "the reduce-scatter GEMM is not batched");
  if (args->out_kind != BSG_OUT_BF16 || args->C || args->beta != 0.0f || args->beta_ptr || args->bias_mode != BSG_BIAS_NONE ||
      args->activation != BSG_ACT_IDENTITY)
    return fail(BSG_ERR_NOT_SUPPORTED, "the reduce-scatter GEMM computes bf16 D = alpha * A B^T only (partial sums travel as bf16)");
  if (args->kind != BSG_KIND_NVFP4 && args->kind != BSG_KIND_MXFP8) return fail(BSG_ERR_NOT_SUPPORTED, "the reduce-scatter GEMM takes NVFP4 or MXFP8 operands");
  bsg_gemm_args local = *args;
  local.batch = 1;
  local.cta_group = 2;
  local.tile_n = 256;
  local.scheduler = BSG_SCHED_STATIC;
  local.use_pdl = 0;
  const uint32_t epoch = c->epoch + 1;
  const int32_t half = int32_t(epoch & 1u);
  uint8_t* out_half = c->base + c->out_off + (half ? size_t(c->M) * size_t(c->N) * 2 : 0);
  if (allreduce) {          // D of the arguments is not used: the result lands in the communicator's output
    local.D = out_half;
    local.ldd = c->N;
  }
  Problem q = from_dense(&local);
  // D holds this rank's slice only; the checks of validate() that look at D's extent use the slice pitch
  q.rs = true;
  q.rs_world = c->world; q.rs_rank = c->rank; q.rs_slice_rows = int32_t(c->slice_rows);
  q.rs_epoch = epoch;
  q.rs_parity = half;
  const int left = (c->rank + c->world - 1) % c->world, right = (c->rank + 1) % c->world;
  q.rs_recv = c->base + c->recv_off;
  q.rs_recv_left = c->peer_base[left] + c->recv_off;
  q.rs_flags = reinterpret_cast<uint32_t*>(c->base + c->flags_off);
  q.rs_flags_left = reinterpret_cast<uint32_t*>(c->peer_base[left] + c->flags_off);
  q.rs_sync = reinterpret_cast<uint32_t*>(c->base + c->sync_off);
  q.rs_sync_left = reinterpret_cast<uint32_t*>(c->peer_base[left] + c->sync_off);
  q.rs_sync_right = reinterpret_cast<uint32_t*>(c->peer_base[right] + c->sync_off);
  if (allreduce) {
    q.rs_allreduce = 1;
    q.rs_out_half = half;
    q.rs_out_maps = c->base + c->maps_off;
    for (int i = 0; i < c->world; ++i) q.rs_peer_sync[i] = reinterpret_cast<uint32_t*>(c->peer_base[i] + c->sync_off);
    // every all-reduce call adds (world - 1) slices x tiles x 8 epilogue warps to the arrival counter
    c->ar_calls += 1;
    q.rs_done_target = uint32_t(c->ar_calls) * uint32_t(c->world - 1) * uint32_t(c->tiles_per_slice * c->tiles_n) * 8u;
  }
  int32_t rc = run_problem(q, workspace, workspace_bytes, cuda_stream);
  if (rc != BSG_OK) { if (allreduce) c->ar_calls -= 1; return rc; }
  c->epoch += 1;
  if (result) *result = out_half;
  return BSG_OK;
}

int32_t bsg_rs_gemm_run(bsg_rs_comm* c, const bsg_gemm_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  return rs_run(c, args, workspace, workspace_bytes, cuda_stream, false, nullptr);
}

int32_t bsg_rs_allreduce_run(bsg_rs_comm* c, const bsg_gemm_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream, void** result) {
  if (!result) return fail(BSG_ERR_INVALID_PROBLEM, "result is null");
  return rs_run(c, args, workspace, workspace_bytes, cuda_stream, true, result);
}

int32_t bsg_rs_destroy(bsg_rs_comm* c) {
  if (!c) return BSG_OK;
  cudaDeviceSynchronize();
  for (int q = 0; q < c->world; ++q) {
    if (c->opened[q]) cudaIpcCloseMemHandle(c->peer_base[q]);
  }
  if (c->base) cudaFree(c->base);
  delete c;
  return BSG_OK;
}

int32_t bsg_tp_set_mode(bsg_tp_comm* c, int32_t mode) {
  if (!c) return fail(BSG_ERR_INVALID_PROBLEM, "null communicator");
  if (mode < 0 || mode > (BSG_TP_PUSH_COPY_ENGINE | BSG_TP_SINGLE_BUFFER | BSG_TP_RELEASE_ANNOUNCE | BSG_TP_PACED_PUSH | BSG_TP_SPREAD_PUSH)) return fail(BSG_ERR_NOT_SUPPORTED, "unknown tensor-parallel mode %d", mode);
  c->mode = mode;
  return BSG_OK;
}

int32_t bsg_tp_destroy(bsg_tp_comm* c) {
  if (!c) return BSG_OK;
  cudaDeviceSynchronize();
  for (int q = 0; q < c->world; ++q) {
    if (c->opened[q]) cudaIpcCloseMemHandle(c->peer_base[q]);
  }
  for (int i = 1; i < 4; ++i) if (c->lanes[i]) cudaStreamDestroy(c->lanes[i]);
  for (int i = 0; i < 4; ++i) if (c->ev_lane[i]) cudaEventDestroy(c->ev_lane[i]);
  if (c->side) cudaStreamDestroy(c->side);
  if (c->ev_start) cudaEventDestroy(c->ev_start);
  if (c->ev_done) cudaEventDestroy(c->ev_done);
  if (c->base) cudaFree(c->base);
  delete c;
  return BSG_OK;
}

}  // extern "C"
