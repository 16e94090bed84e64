/*
 * bsgemm.h -- C ABI of the Blackwell (sm_100a) block-scaled GEMM library.
 *
 * Plain C, plain pointers and sizes.  Every entry point returns a bsg_status
 * (0 = success) and never throws, aborts or allocates unless stated.  All
 * device pointers are ordinary CUDA device pointers owned by the caller; work
 * is enqueued on the given stream and the call returns without synchronising.
 *
 * Each entry point names the interface of the reference library (NVIDIA
 * CUTLASS, paths relative to its source tree) whose role it takes over.
 */
#ifndef BSGEMM_H_
#define BSGEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes, modelled on cutlass::Status (include/cutlass/cutlass.h). */
typedef enum bsg_status {
  BSG_OK = 0,
  BSG_ERR_MISALIGNED_OPERAND = 1,
  BSG_ERR_INVALID_PROBLEM = 2,
  BSG_ERR_NOT_SUPPORTED = 3,
  BSG_ERR_WORKSPACE_NULL = 4,
  BSG_ERR_INTERNAL = 5,
  BSG_ERR_ARCH_MISMATCH = 6,
  BSG_ERR_TIMEOUT = 7,      /* a bounded device-side wait ran out */
  BSG_ERR_CUDA = 8
} bsg_status;

/* Operand formats (data format of A and B, and the scale format that goes with it). */
enum {
  BSG_KIND_NVFP4 = 0,       /* e2m1 data, ue4m3 scale per 16 K-elements */
  BSG_KIND_MXFP8 = 1,       /* e4m3 data, ue8m0 scale per 32 K-elements */
  BSG_KIND_MXFP4 = 2,       /* e2m1 data, ue8m0 scale per 32 K-elements */
  BSG_KIND_MXFP8_MXFP4 = 3  /* A e4m3, B e2m1 (packed, 32-byte aligned), both with ue8m0 scale per 32: the mixed form of the
                               reference's examples/72_blackwell_narrow_precision_gemm/72c_blackwell_mixed_mxfp8_bf16_gemm.cu;
                               K must be a multiple of 128.  Kinds 2 and 3: cta_group 2, static scheduler, not tensor parallel. */
};

/* Output formats. */
enum {
  BSG_OUT_BF16 = 0,         /* D = bf16(alpha*acc + beta*C) */
  BSG_OUT_NVFP4 = 1,        /* D = e2m1 packed + SFD ue4m3 per 16 N-elements, interleaved layout */
  BSG_OUT_MXFP8 = 2,        /* D = e4m3 + SFD ue8m0 (round-up conversion) per 32 N-elements, interleaved layout */
  BSG_OUT_F16 = 3,          /* D = fp16(...)  (C, when given, stays bf16) */
  BSG_OUT_F32 = 4,          /* D = fp32(...): the epilogue's own precision, nothing rounded */
  BSG_OUT_E4M3 = 5,         /* D = e4m3(...) without scale factors: round to nearest even, saturating at +-448, NaN -> 0x7F */
  BSG_OUT_E5M2 = 6          /* D = e5m2(...) likewise, saturating at +-57344 (infinity too) */
};

/*
 * Arguments of one dense (optionally batched) block-scaled GEMM
 *     D[l] = alpha * (A[l] . SFA[l]) (B[l] . SFB[l])^T + beta * C[l].
 * Field-for-field stand-in for cutlass::library::BlockScaledGemmArguments
 * (tools/library/include/cutlass/library/library.h:354-397).
 *
 * A is (batch, M, K) and B is (batch, N, K), both K-major (two e2m1 per byte,
 * even K index in the low nibble); rows may carry a pitch (lda / ldb) and batch
 * entries a stride, so a slice of a larger buffer can be passed as it is.
 * SFA / SFB use the 128-row x 4-K-block interleaved layout of
 * include/cutlass/detail/sm100_blockscaled_layout.hpp:49-114, one layout per
 * batch entry, padding included (the reference derives that layout from the
 * shape alone: it has no strides).  C and D are (batch, M, N) row-major.
 */
/* Element-wise activation applied to alpha * acc + bias + beta * C before the output conversion / quantisation
 * (include/cutlass/epilogue/thread/activation.h of the reference: ReLu :145, GELU<float> :585, SiLu :452). */
typedef enum bsg_activation { BSG_ACT_IDENTITY = 0, BSG_ACT_RELU = 1, BSG_ACT_GELU = 2, BSG_ACT_SILU = 3 } bsg_activation;
/* Which output coordinate indexes the bias vector (PerColumnBias of the reference's host epilogue,
 * tools/util/include/cutlass/util/reference/host/gett.hpp:189,717). */
typedef enum bsg_bias_mode { BSG_BIAS_NONE = 0, BSG_BIAS_PER_COLUMN = 1, BSG_BIAS_PER_ROW = 2 } bsg_bias_mode;

typedef struct bsg_gemm_args {
  int32_t kind;             /* BSG_KIND_* */
  int32_t out_kind;         /* BSG_OUT_* */
  int32_t batch;            /* L >= 1 */
  int32_t reserved0;
  int64_t M, N, K;          /* logical extents (K in elements) */
  const void* A;
  const void* B;
  const void* SFA;
  const void* SFB;
  const void* C;            /* bf16, may be NULL when beta == 0 */
  void* D;                  /* bf16; packed e2m1 (BSG_OUT_NVFP4); e4m3 (BSG_OUT_MXFP8); fp16; fp32; e4m3 / e5m2 */
  void* SFD;                /* scale factors of D, interleaved over (M, N/16) or (M, N/32); quantised outputs only */
  int64_t ldc;              /* C row pitch in elements (0 = N) */
  int64_t ldd;              /* D row pitch in elements (0 = N) */
  float alpha;
  float beta;
  const float* alpha_ptr;   /* optional device scalars, override alpha / beta */
  const float* beta_ptr;
  const float* norm_constant; /* device fp32 scalar: required for BSG_OUT_NVFP4, optional (NULL = 1) for BSG_OUT_MXFP8 */
  int32_t tile_n;           /* 0 = library default (256, or 128 when N <= 128), else 64, 128, 192 or 256; 64 and 192: NVFP4 / MXFP8,
                               cta_group 2, static scheduler, bf16 or re-quantised row-major output */
  int32_t cta_group;        /* 0 = default, else 1 or 2 (CTAs per MMA) */
  int32_t sm_count;         /* 0 = all SMs of the current device */
  int32_t raster_band;      /* 0 = default band height in tiles */
  /* D = act(alpha * acc + bias + beta * C), the reference's order of operations (gett.hpp:714-761). */
  const float* bias;        /* device fp32: N entries (per column) or M entries (per row), shared by all batches; or NULL */
  int32_t bias_mode;        /* BSG_BIAS_* (BSG_BIAS_NONE ignores bias) */
  int32_t activation;       /* BSG_ACT_* */
  /* Strides in ELEMENTS, 0 = densely packed (library.h:374-383: lda, ldb, batch_stride_A..D).  lda / ldb must keep
   * every row 16-byte aligned (multiples of 32 for e2m1, of 16 for e4m3). */
  int64_t lda;              /* A row pitch (0 = K) */
  int64_t ldb;              /* B row pitch (0 = K) */
  int64_t batch_stride_A;   /* elements between A[l] and A[l+1] (0 = M * lda) */
  int64_t batch_stride_B;   /* (0 = N * ldb) */
  int64_t batch_stride_C;   /* (0 = M * ldc) */
  int64_t batch_stride_D;   /* (0 = M * ldd) */
  int32_t use_pdl;          /* 1: launch with programmatic stream serialisation (library.h:396 use_pdl): the kernel's
                               set-up overlaps the tail of the previous kernel on the stream and it waits
                               (griddepcontrol.wait) before its first global access */
  int32_t scheduler;        /* BSG_SCHED_* */
  /* cluster_shape / cluster_shape_fallback of the reference (library.h:357-358).  The kernels here use no TMA
   * multicast, so the cluster is exactly the CTA group of one MMA and there is no larger preferred shape to fall
   * back from: 0 (default) or {cta_group, 1} are accepted, anything else is BSG_ERR_NOT_SUPPORTED. */
  int32_t cluster_m, cluster_n;
  int32_t cluster_fallback_m, cluster_fallback_n;
  int32_t out_layout;       /* BSG_LAYOUT_*: quantised outputs only, batch 1 */
  int32_t reserved1;
} bsg_gemm_args;

/* Layout of a quantised output.  ROW_MAJOR: D is (M, N) with N contiguous, one scale factor per 16 / 32 consecutive
 * columns of a row, SFD interleaved over (M, N / V).  COL_MAJOR: D is stored column-major -- (N, M) with M contiguous,
 * ldd its pitch in elements -- with one scale factor per 16 / 32 consecutive ROWS of a column and SFD interleaved over
 * (N, M / V): the K-major operand form of D^T, which a following GEMM can take as its B with K := M (the reference's
 * Sm100BlockScaleFactorColStore, include/cutlass/epilogue/fusion/sm100_visitor_store_tma_warpspecialized.hpp:352, and the
 * M-major layout of Sm1xxBlockScaledOutputConfig, include/cutlass/detail/sm100_blockscaled_layout.hpp:192-228).  M must be a
 * multiple of 32. */
enum { BSG_LAYOUT_ROW_MAJOR = 0, BSG_LAYOUT_COL_MAJOR = 1 };

/* Tile schedulers.  STATIC: persistent grid of one cluster per SM pair, tile index += cluster count (the
 * reference's StaticPersistentTileScheduler, python/CuTeDSL/cutlass/utils/static_persistent_tile_scheduler.py:376).
 * DYNAMIC: one cluster per output tile is launched and every running cluster, when it has finished a tile, cancels a
 * not-yet-started cluster and takes over its tile (clusterlaunchcontrol.try_cancel; the reference's
 * PersistentTileSchedulerSm100, include/cutlass/gemm/kernel/sm100_tile_scheduler.hpp:400-423), so tiles are handed
 * out in the order clusters become free and the GPU can be shared with other kernels. */
enum { BSG_SCHED_STATIC = 0, BSG_SCHED_DYNAMIC = 1 };

/*
 * Arguments of a grouped (MoE) GEMM with ragged M: the rows of all groups are
 * contiguous in A and D, group g owns rows [offsets[g-1], offsets[g]) and its
 * own B[g] (N x K) and SFB[g].  SFA holds one interleaved layout per group,
 * back to back, each padded to 128 rows.  Mirrors
 * cutlass::library::GroupedGemmBlockScaledArguments
 * (tools/library/include/cutlass/library/library.h:558-605) in its
 * contiguous-token form (MoEProblemShape,
 * include/cutlass/gemm/group_array_problem_shape.hpp:85-131) and the Python
 * GroupedGemmArguments.offsets contract
 * (operators/cutlass/operators/arguments/grouped_gemm.py:59-86).
 */
typedef struct bsg_grouped_args {
  int32_t kind;
  int32_t out_kind;         /* BSG_OUT_*; quantised outputs need SFD (and norm_constant for NVFP4) below */
  int32_t num_groups;       /* 1..BSG_MAX_GROUPS */
  int32_t reserved0;
  int64_t total_M;          /* rows of A and D (sum of group sizes) */
  int64_t N, K;
  const void* A;            /* (total_M, K) */
  const void* B;            /* (num_groups, N, K) */
  const void* SFA;
  const void* SFB;
  const void* C;            /* (total_M, N) bf16 or NULL */
  void* D;                  /* (total_M, N): bf16, packed e2m1 or e4m3 */
  const int32_t* offsets;   /* device int32[num_groups], cumulative END rows */
  int64_t ldc, ldd;
  float alpha, beta;
  int32_t tile_n, cta_group, sm_count, raster_band;
  const float* bias;        /* device fp32 (num_groups, N): one vector per group, added per output column; or NULL */
  int32_t reserved1;
  int32_t activation;       /* BSG_ACT_* */
  const float* alpha_array; /* device fp32[num_groups]: one alpha per group, overrides alpha; or NULL.  The reference passes
                               per-group scalars as pointer arrays (examples/75_blackwell_grouped_gemm_block_scaled/
                               75_blackwell_grouped_gemm_block_scaled.cu:693-719) */
  const float* beta_array;  /* likewise for beta */
  /* Quantised output per group (the reference's grouped block-scaled example emits SFD per group,
   * examples/75_blackwell_grouped_gemm/75_blackwell_grouped_gemm_block_scaled.cu:551-566): SFD holds one interleaved
   * layout over (M_g, N/16 or N/32) per group, back to back, each padded to 128 rows -- the form SFA has, so the
   * output feeds the next grouped GEMM (K := N) as it is.  Pad rows of a group's last atom are not written. */
  void* SFD;
  const float* norm_constant; /* device fp32 scalar shared by all groups */
  int32_t use_pdl;
  int32_t scheduler;        /* BSG_SCHED_* */
} bsg_grouped_args;

#define BSG_MAX_GROUPS 256

typedef struct bsg_caps {
  int32_t tile_m, tile_n, tile_k;   /* MMA tile chosen for these arguments */
  int32_t cta_group;
  int32_t stages;                   /* shared-memory pipeline depth */
  int32_t smem_bytes;
  int64_t num_tiles;                /* -1 when only known on the device (grouped) */
} bsg_caps;

/* Library version as major*10000 + minor*100 + patch. */
int32_t bsg_version(void);

/* Text of the last error raised on the calling thread (never NULL). */
const char* bsg_last_error_string(void);

/* Can these arguments run?  Fills caps when non-NULL.  Replaces
 * GemmUniversalAdapter::can_implement (include/cutlass/gemm/device/gemm_universal_adapter.h:232)
 * and Operator.supports (operators/cutlass/operators/base.py:126). */
int32_t bsg_gemm_query(const bsg_gemm_args* args, bsg_caps* caps);
int32_t bsg_grouped_query(const bsg_grouped_args* args, bsg_caps* caps);

/* Bytes of device workspace a run needs (a status word; small).  Replaces
 * GemmUniversalAdapter::get_workspace_size (gemm_universal_adapter.h:243). */
int32_t bsg_gemm_workspace_size(const bsg_gemm_args* args, size_t* bytes);
int32_t bsg_grouped_workspace_size(const bsg_grouped_args* args, size_t* bytes);

/* Zero a fresh workspace (asynchronously, on the stream) before its first use.  Takes the
 * place of GemmUniversalAdapter::initialize's workspace set-up (gemm_universal_adapter.h:313)
 * and Operator.initialize_workspace (operators/cutlass/operators/base.py:208). */
int32_t bsg_workspace_init(void* workspace, size_t workspace_bytes, void* cuda_stream);

/* Enqueue the GEMM; nothing else is put on the stream.  The workspace must have been
 * initialised once (bsg_workspace_init) and stay alive until the stream reaches the end of
 * the kernel; its first word accumulates a device-side status over all runs until it is
 * read (see bsg_read_device_status).  Replaces GemmUniversalAdapter::run
 * (gemm_universal_adapter.h:375) and Operator.run (operators/cutlass/operators/base.py:165). */
int32_t bsg_gemm_run(const bsg_gemm_args* args, void* workspace, size_t workspace_bytes,
                     void* cuda_stream);
int32_t bsg_grouped_run(const bsg_grouped_args* args, void* workspace, size_t workspace_bytes,
                        void* cuda_stream);

/* Synchronise the stream, translate the workspace status word (0 -> BSG_OK, a timed-out
 * device-side wait -> BSG_ERR_TIMEOUT, bad group offsets -> BSG_ERR_INVALID_PROBLEM) and
 * clear it. */
int32_t bsg_read_device_status(void* workspace, void* cuda_stream);

/*
 * Grouped GEMM in the pointer-array form: every group is a problem of its own -- its own (M, N, K), its own A, B,
 * SFA, SFB, C, D (and SFD) tensors with their own row pitches.  Mirrors cutlass::library::GroupedGemmBlockScaledArguments
 * with GroupProblemShape (tools/library/include/cutlass/library/library.h:558-605,
 * include/cutlass/gemm/group_array_problem_shape.hpp:55-83; device-side tensor-map updates in
 * include/cutlass/gemm/collective/sm100_blockscaled_mma_array_warpspecialized.hpp:1142-1343).
 *
 * Difference to the reference, which keeps its pointer arrays in device memory and rewrites one tensor map per
 * operand on the device whenever a CTA moves to another group: here the problem sizes and pointer arrays are HOST
 * arrays (the reference passes a host copy of the sizes too, problem_sizes_3x_host).  bsg_ptr_array_initialize encodes
 * five tensor maps per group on the host and uploads them, with the extents, as one table into the workspace; the
 * kernel reads a group's maps from that table.  bsg_ptr_array_run only launches.  A caller that holds device arrays
 * copies them to the host once, where the reference's Operation::initialize runs (library.h:547-556).
 *
 * Per group g: A_g is (M_g, K_g) K-major with pitch lda[g], B_g is (N_g, K_g) with pitch ldb[g], SFA_g / SFB_g are
 * interleaved layouts over (M_g, K_g / V) and (N_g, K_g / V), C_g / D_g are (M_g, N_g) with pitches ldc[g] / ldd[g],
 * SFD_g an interleaved layout over (M_g, N_g / V_out).  Alignment rules per group are those of bsg_gemm_args.
 * Groups with M_g == 0 or N_g == 0 are skipped.  Static scheduler, cta_group 2, row-major outputs.
 */
typedef struct bsg_ptr_array_args {
  int32_t kind;                 /* BSG_KIND_NVFP4 or BSG_KIND_MXFP8 */
  int32_t out_kind;             /* BSG_OUT_* */
  int32_t num_groups;           /* 1..BSG_MAX_GROUPS */
  int32_t activation;           /* BSG_ACT_* */
  const int32_t* problem_sizes; /* HOST int32[num_groups][3]: M, N, K of every group */
  const void* const* A;         /* HOST arrays of num_groups device pointers each */
  const void* const* B;
  const void* const* SFA;
  const void* const* SFB;
  const void* const* C;         /* or NULL (no C anywhere); single entries may be NULL too */
  void* const* D;
  void* const* SFD;             /* quantised outputs only, else NULL */
  const int64_t* lda;           /* HOST int64[num_groups], elements; NULL: packed (K_g, K_g, N_g, N_g) */
  const int64_t* ldb;
  const int64_t* ldc;
  const int64_t* ldd;
  float alpha, beta;
  const float* alpha_array;     /* device fp32[num_groups] or NULL, as in bsg_grouped_args */
  const float* beta_array;
  const float* norm_constant;   /* device fp32 scalar (NVFP4 output) */
  int32_t tile_n;               /* 0 = auto, 128 or 256 */
  int32_t sm_count;
  int32_t raster_band;
  int32_t use_pdl;
} bsg_ptr_array_args;

/* Workspace: the status word plus the per-group table (768 bytes per group). */
int32_t bsg_ptr_array_workspace_size(const bsg_ptr_array_args* args, size_t* bytes);
/* Checks every group, encodes its tensor maps and copies the table into the workspace (on the stream; the host
 * arrays may be released when the call returns).  Call again whenever a pointer, size or pitch changes. */
int32_t bsg_ptr_array_initialize(const bsg_ptr_array_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream);
/* The same for a caller whose arrays are where the reference keeps them, in DEVICE memory (ptr_A ... ptr_D, the pitches
 * and problem_sizes_3x of library.h:558-605): every non-null array member of `args` is then a device pointer.  The
 * arrays are copied to the host first (the stream is synchronised), after which this is bsg_ptr_array_initialize; a later
 * bsg_ptr_array_run wants problem_sizes readable on the host (the reference passes problem_sizes_3x_host as well). */
int32_t bsg_ptr_array_initialize_from_device(const bsg_ptr_array_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream);
/* Launches the grouped GEMM described by the table that bsg_ptr_array_initialize left in this workspace; of `args`
 * the scalars (alpha, beta and their arrays, norm_constant, activation, use_pdl) and the problem sizes are read. */
int32_t bsg_ptr_array_run(const bsg_ptr_array_args* args, void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * The same dense / batched GEMM as bsg_gemm_run for callers that have no device memory to hand over
 * as workspace and are not allowed to create any: code running under a framework that has frozen or
 * pre-reserved all device memory (an inference server after warm-up, a plug-in whose enqueue hook
 * may not call the allocator), or code sitting inside a region where cudaMalloc is forbidden.
 * Nothing is allocated, by this call or by anything it calls.  The kernel's scratch (its status
 * word) lives in a 256-byte array that is part of the library image on every GPU that loads it;
 * a problem whose scratch need exceeds those 256 bytes is refused with BSG_ERR_NOT_SUPPORTED.
 *
 *  - The first call on each device looks the array's address up (one-time set-up, with that device
 *    current).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array.  Each call clears the part it uses before its
 *    kernel runs, so results do not depend on earlier calls; but two calls whose kernels can overlap
 *    on the GPU (different streams) race on it -- keep calls to this entry point on one stream, or
 *    otherwise ordered.
 *  - device_status_out may be NULL.  If it is not, the call waits for the stream, stores the kernel's status
 *    word there (0 = every device-side wait completed) and returns BSG_ERR_TIMEOUT when it is not 0, as
 *    bsg_read_device_status does; a waiting call like that does not belong inside a stream capture.  With NULL
 *    nobody reads the word: the next call's clearing erases it, so a time-out goes unnoticed (the sticky word of
 *    a caller-provided workspace has no such gap).
 *  - Arguments are checked before anything is enqueued: a refused call leaves the stream and the array untouched.
 *  - The address that was looked up belongs to the device's current context; it does not survive cudaDeviceReset.
 *
 * This entry point has no counterpart in the reference; it exists for such callers only.
 */
int32_t bsg_gemm_run_static(const bsg_gemm_args* args, void* cuda_stream, uint32_t* device_status_out);

/*
 * Block-scaled quantiser: the step in front of the GEMM that turns a bf16 matrix X (rows x K,
 * row-major) into a GEMM operand -- quantised values plus scale factors already in the interleaved
 * layout (512-byte atoms of 128 rows x 4 K-blocks) that bsg_gemm_args.SFA / SFB expect.
 * The reference leaves this step to the caller ("a quantization step or an earlier kernel",
 * operators/examples/006_block_scaled_gemm.ipynb; layout contract
 * operators/cutlass/operators/arguments/operand.py:353-367); the arithmetic is the one of its
 * block-scale epilogue (tools/util/include/cutlass/util/reference/host/gett.hpp:436-478): per row and
 * K-block, amax -> SF = cvt(amax * (st / fp_max)) -> q = cvt(x * min(st / float(SF), FLT_MAX)).
 *   kind BSG_KIND_NVFP4: K-blocks of 16, SF ue4m3, values e2m1 packed two per byte (Q is rows x K/2 bytes);
 *   kind BSG_KIND_MXFP8: K-blocks of 32, SF ue8m0 (conversion rounds up), values e4m3 (Q is rows x K bytes).
 * SF receives whole atoms: ceil(rows/128) * ceil(K/V/4) * 512 bytes, zero where no row / K-block exists.
 * norm_constant: device fp32 scalar st (NVFP4: typically 448 * 6 / amax of X; MXFP8: 1), NULL = 1.0.
 * K must be a multiple of 32, ldx (in elements, >= K) a multiple of 8, all pointers 16-byte aligned.
 * Asynchronous on cuda_stream; allocates nothing.
 */
typedef struct bsg_quant_args {
  int32_t kind;
  int32_t use_pdl;          /* 1: launched as a programmatic dependent launch (as bsg_gemm_args.use_pdl): the kernel's set-up
                               overlaps the tail of the kernel before it on the stream, and a GEMM launched with use_pdl behind
                               it starts its own set-up while this one drains */
  int64_t rows, K;
  const void* X;
  int64_t ldx;
  void* Q;
  void* SF;
  const float* norm_constant;
} bsg_quant_args;
int32_t bsg_quantize(const bsg_quant_args* args, void* cuda_stream);

/*
 * Tensor-parallel GEMM: D[:, local N shard] = alpha * A B_local^T + beta * C, with A (and SFA)
 * sharded by rows over `world` ranks (one process per GPU of one node) and B / D sharded over N.
 * The kernel itself gathers A over NVLink: a push warp in every CTA sends this rank's rows into the
 * peers' buffers (bulk copies through shared memory, nearest consumer first) and bumps a per-row-block
 * counter there, while the tensor-core warps already work on the rows that have arrived.
 * Takes the role of the reference's all-gather distributed GEMM
 * (include/cutlass/experimental/distributed/device/dist_gemm_universal_wrapper.hpp:53,
 * schedule AllGather1D_TilingCD_RotatingA in schedules/dist_gemm_1d_schedules.hpp; device barrier
 * kernel/full_barrier.hpp:47), with bounded waits instead of unbounded spins.
 *
 * bsg_tp_create   allocates this rank's buffers (two full-size gathered A and SFA buffers, used by
 *                 alternate calls so that a peer may already send the next call's rows while this rank
 *                 still computes, plus sync words; the only allocating call) and returns a 64-byte
 *                 CUDA IPC handle to hand to the peers.
 * bsg_tp_connect  takes the `world` handles (64 bytes each, indexed by rank) and maps the peers.
 * bsg_tp_buffers  returns where this rank writes its own A / SFA shard (a_shard, sfa_shard: inside the
 *                 first gathered buffer, whose start is a_full / sfa_full; the other ranks' rows of that
 *                 buffer are filled by every second call only, so read a_full for
 *                 diagnosis, not as an output).
 * bsg_tp_gemm_run enqueues one GEMM; args->A / SFA are ignored, args->M is the full M, args->N
 *                 the local N shard.  All ranks must call it the same number of times with the
 *                 same shapes.
 *                 The caller may rewrite its shard for the next call as soon as this call is complete on the
 *                 stream (the push has read it by then).  With the default two gathered buffers a rank may run
 *                 at most one call ahead of its slowest peer; the device-side waits that enforce this are
 *                 bounded (about two seconds), after which bsg_read_device_status reports BSG_ERR_TIMEOUT.
 * bsg_tp_destroy  frees the buffers the peers write into: call it only after every rank has finished its last
 *                 call (synchronise the device, then a barrier across the ranks), never with a call in flight.
 * bsg_tp_set_mode  chooses who moves the shard: BSG_TP_PUSH_KERNEL -- a warp of the GEMM kernel itself, through
 *                 the SM's bulk-copy engine (one launch per GEMM); or
 *                 BSG_TP_PUSH_COPY_ENGINE -- the GPU's copy engines on an internal side stream, one transfer per
 *                 band of row blocks followed by its announcement, joined back into the caller's stream
 *                 (the scheme of dist_gemm_universal_wrapper.hpp:578-593).  Default: kernel.  All ranks must use the same mode.
 *
 * A call needs the whole GPU.  Every CTA of a launch pushes pieces that a peer's CTAs wait for, so all CTAs of all
 * ranks must be resident at the same time: the grid is sized from the number of clusters that fit (asked once per
 * device), but another kernel that occupies SMs while a call runs (a second stream, another process under MPS) can
 * leave CTAs unscheduled and the ranks waiting for one another until the bounded waits give up (BSG_ERR_TIMEOUT).
 * After BSG_ERR_TIMEOUT the arrival counters of the ranks are out of step: destroy the communicators on all ranks
 * (bsg_tp_destroy after a device synchronise and a barrier) and create them again before the next call.
 *
 * Ordering of the announcements.  A piece is announced to the peer by a system-scope counter increment issued after
 * cp.async.bulk.wait_group has reported the piece's stores complete; the peer acquires the counter and issues a proxy
 * fence before its TMA loads.  With BSG_TP_RELEASE_ANNOUNCE (part of the default mode) a proxy fence and a system-scope
 * release fence stand in front of every batch of increments: the form the PTX memory model asks for.  Without it the
 * increment is relaxed and nothing but the way bulk stores complete over NVLink keeps it behind the data: faster, and
 * seen to fail on 8 GPUs (a rank read a row block before its rows had landed, in a run of many small calls).
 */
enum { BSG_TP_PUSH_KERNEL = 0, BSG_TP_PUSH_COPY_ENGINE = 1, BSG_TP_SINGLE_BUFFER = 2 /* or-ed in: every call uses the first gathered buffer */,
       BSG_TP_RELEASE_ANNOUNCE = 4 /* or-ed in: see "Ordering of the announcements" above */,
       BSG_TP_PACED_PUSH = 8 /* or-ed in: a CTA pushes the rows for its j-th nearest consumer while it works on stage j - 1 of
                                its own walk (they arrive a stage before they are needed) instead of everything at once */,
       BSG_TP_SPREAD_PUSH = 16 /* or-ed in: as BSG_TP_PACED_PUSH, with the pieces of a stage leaving evenly over the first three
                                 quarters of that stage instead of in one burst at its start */ };
typedef struct bsg_tp_comm bsg_tp_comm;
/* A new communicator starts in BSG_TP_PUSH_KERNEL | BSG_TP_SPREAD_PUSH | BSG_TP_RELEASE_ANNOUNCE; bsg_tp_set_mode replaces the whole mode word (0 = the
 * kernel pushes everything as fast as the links allow).  Only between calls, with every rank idle, the same on all ranks. */
int32_t bsg_tp_set_mode(bsg_tp_comm* comm, int32_t mode);
int32_t bsg_tp_create(int32_t rank, int32_t world, int32_t kind, int64_t M, int64_t K, bsg_tp_comm** out,
                      void* ipc_handle_out);
int32_t bsg_tp_connect(bsg_tp_comm* comm, const void* all_handles);
int32_t bsg_tp_buffers(bsg_tp_comm* comm, void** a_full, void** sfa_full, void** a_shard, void** sfa_shard);
int32_t bsg_tp_gemm_run(bsg_tp_comm* comm, const bsg_gemm_args* args, void* workspace, size_t workspace_bytes,
                        void* cuda_stream);
int32_t bsg_tp_destroy(bsg_tp_comm* comm);

/*
 * GEMM + reduce-scatter: the row-parallel half of a tensor-parallel layer.  K is sharded: every rank holds
 * A[:, its K shard] (M x K/world) and B[:, its K shard] (N x K/world) with their scale factors and computes a partial
 * product for all of M x N; the partial sums are reduced over the ranks and scattered over M: rank r ends up with rows
 * [r * M / world, (r + 1) * M / world) of D = alpha * A B^T.  One kernel per rank does both: the M tiles are walked
 * slice by slice (a slice = the rows one rank owns), starting at slice rank + 1; the epilogue of a tile adds the partial
 * sums received from rank + 1 (none in the first stage), and stores the sum into the receive buffer of rank - 1 (TMA
 * stores into peer memory, then a released counter increment per warp), or, in the last stage, into D.  Takes the role
 * of the reference's ReduceScatter1D_TilingA_RotatingC schedule
 * (include/cutlass/experimental/distributed/schedules/dist_gemm_1d_schedules.hpp:148), in which the running sums also
 * travel around the ring in the output type: here bf16, rounded at every hop, fp32 only inside a hop.
 *
 * bsg_rs_create    allocates the receive buffers (two halves, used by alternate calls; (world - 1) * M / world * N bf16
 *                  each) and returns a 64-byte CUDA IPC handle for the peers.  M a multiple of 256 * world.
 * bsg_rs_connect   takes the `world` handles (64 bytes each, by rank) and maps the two ring neighbours (all ranks with
 *                  BSG_RS_WITH_ALLREDUCE).
 * bsg_rs_gemm_run  enqueues one GEMM: args->M, N are the full extents, K the local shard, A / B / SFA / SFB the local
 *                  shards, D the (M / world) x N bf16 result slice of this rank (ldd its pitch); alpha applies to every
 *                  partial product; C, beta, bias, activation and quantised outputs are not available.  All ranks call
 *                  it the same number of times; waits are bounded as for the all-gather GEMM (BSG_ERR_TIMEOUT), and the
 *                  same rules hold for what a call needs (the whole GPU) and for recovery after a time-out.
 * bsg_rs_allreduce_run  GEMM + all-reduce (communicators created with BSG_RS_WITH_ALLREDUCE): the same ring, but the
 *                  epilogue of the last stage stores the finished slice into the full-size output of EVERY rank (TMA
 *                  stores into peer memory, a released counter increment per warp and destination), and the kernel ends
 *                  only once the slices of all other ranks have arrived, so the next kernel on the stream finds all of
 *                  D = alpha * A B^T.  The output (M x N bf16, pitch N) belongs to the communicator, which holds two of
 *                  them for alternate calls: *result points at the one this call fills, valid until the call after the
 *                  next one is enqueued.  args->D is not used.  (The reference's schedules stop at the reduce-scatter;
 *                  this is that schedule followed by the all-gather of its result, inside the same kernel.)
 * bsg_rs_destroy   after the device is idle on every rank and a barrier.
 */
typedef struct bsg_rs_comm bsg_rs_comm;
enum { BSG_RS_WITH_ALLREDUCE = 1 };   /* flags of bsg_rs_create: also allocate the two M x N outputs of bsg_rs_allreduce_run */
int32_t bsg_rs_create(int32_t rank, int32_t world, int64_t M, int64_t N, int32_t flags, bsg_rs_comm** out, void* ipc_handle_out);
int32_t bsg_rs_connect(bsg_rs_comm* comm, const void* all_handles);
int32_t bsg_rs_gemm_run(bsg_rs_comm* comm, const bsg_gemm_args* args, void* workspace, size_t workspace_bytes,
                        void* cuda_stream);
int32_t bsg_rs_allreduce_run(bsg_rs_comm* comm, const bsg_gemm_args* args, void* workspace, size_t workspace_bytes,
                             void* cuda_stream, void** result);
int32_t bsg_rs_destroy(bsg_rs_comm* comm);

#ifdef __cplusplus
}
#endif
#endif /* BSGEMM_H_ */
