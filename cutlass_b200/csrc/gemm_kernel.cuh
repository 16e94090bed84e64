// Persistent warp-specialised block-scaled GEMM for sm_100a.
//
//   X = act(alpha * (A . SFA)(B . SFB)^T + bias + beta * C)
//   D = bf16(X),  or  (D, SFD) = block-scaled quantisation of X (e2m1 + ue4m3 per 16, or e4m3 + ue8m0 per 32)
//
// One kernel serves the dense, batched, grouped (ragged M) and flag-gated
// (tensor-parallel) forms: every output tile belongs to a "group" that owns a
// contiguous run of rows of A and D, one B matrix and one pair of scale-factor
// layouts.
//
// Roles (192 threads): warps 0-3 epilogue (TMEM lane quadrant = warp id),
// warp 4 UMMA issue + TMEM allocation, warp 5 TMA producer; the tensor-parallel
// variant adds warp 6, which pushes this rank's rows of A to the peers.  With
// CG == 2 two CTAs of a cluster form one 256-row MMA (cta_group::2): both load
// their half of A and B, the even CTA issues the MMA, both run their own epilogue.
//
// The producer and MMA warps run their loops with all 32 lanes (warp-uniform
// control flow and operands; only the issuing instructions are predicated on one
// elected lane), which keeps descriptors and addresses in uniform registers.
//
// This takes the place of the reference kernel
// include/cutlass/gemm/kernel/sm100_gemm_tma_warpspecialized.hpp together with the
// mainloop include/cutlass/gemm/collective/sm100_blockscaled_mma_warpspecialized.hpp
// (load :879, mma :949) and the linear-combination / block-scale-factor epilogue
// (include/cutlass/epilogue/fusion/sm100_visitor_store_tma_warpspecialized.hpp:226-275).
// Every wait is bounded: on a timeout the role records a status bit, issues no further
// loads, MMAs or pushes, runs through its remaining loop iterations with short waits,
// and the kernel returns after a pause for what is still in flight.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cfloat>
#include <cstdint>

#include "ptx.cuh"

namespace bsg {

constexpr int kMaxGroups = 256;
constexpr int kKindNvfp4 = 0;        // e2m1 x e2m1, ue4m3 scale per 16
constexpr int kKindMxfp8 = 1;        // e4m3 x e4m3, ue8m0 scale per 32
constexpr int kKindMxfp4 = 2;        // e2m1 x e2m1, ue8m0 scale per 32
constexpr int kKindMxfp8Mxfp4 = 3;   // A e4m3, B e2m1 (spread by the TMA engine into the 16-byte groups kind::mxf8f6f4 reads), ue8m0 per 32
__host__ __device__ constexpr bool kind_packs_fp4(int kind) { return kind == kKindNvfp4 || kind == kKindMxfp4; }   // A and B: two values per byte
constexpr int kOutBf16 = 0;
constexpr int kOutNvfp4 = 1;
constexpr int kOutMxfp8 = 2;
constexpr int kOutF16 = 3;
constexpr int kOutF32 = 4;
constexpr int kOutE4m3 = 5;      // e4m3 / e5m2 values without scale factors (saturating conversion)
constexpr int kOutE5m2 = 6;
__host__ __device__ constexpr bool out_is_quantised(int out_kind) { return out_kind == kOutNvfp4 || out_kind == kOutMxfp8; }
constexpr int kActIdentity = 0, kActRelu = 1, kActGelu = 2, kActSilu = 3;

// Bits of the device status word.
constexpr uint32_t kStTimeoutFull = 1u;       // MMA warp: operands never arrived
constexpr uint32_t kStTimeoutEmpty = 2u;      // producer: stage never released
constexpr uint32_t kStTimeoutTmemFull = 4u;   // epilogue: accumulator never completed
constexpr uint32_t kStTimeoutTmemEmpty = 8u;  // MMA warp: accumulator never drained
constexpr uint32_t kStTimeoutFlag = 16u;      // producer: row-ready flag never set
constexpr uint32_t kStBadOffsets = 32u;       // grouped: offsets not monotone / out of range

// Pointer-array grouped form (kernel template PTR == true): every group is a problem of its own, with its own
// extents, tensors and tensor maps.  The host encodes one record per group and uploads the array; the kernel reads the
// maps from global memory (after a tensor-map proxy fence) and the extents into its group table.
struct alignas(128) GroupDesc {
  CUtensorMap tmA, tmB, tmSFA, tmSFB, tmD;
  int32_t M, N, K, pad;
  const __nv_bfloat16* C;
  void* D;
  uint8_t* SFD;
  int64_t ldc, ldd;      // elements
};
static_assert(sizeof(GroupDesc) == 768, "group record size is part of the workspace contract");

struct GemmParams {
  int32_t num_groups;         // 1 for a dense GEMM
  int32_t rows_per_group;     // dense / batched: M of every group (offsets == nullptr)
  int32_t total_rows;         // rows of A and D over all groups
  int32_t N, K;
  const int32_t* offsets;     // grouped: cumulative END row of each group (device)
  int32_t b_per_group;        // 1: group g reads B[g] (third coordinate of the B map); 0: one B for all groups
  int32_t sfb_atoms_per_group;
  int32_t batched;            // 1: A, C and D are addressed per group (row within the group; the group is the third
                              //    tensor-map coordinate and selects the batch stride); 0: rows run over all groups
  int64_t batch_stride_c, batch_stride_d;   // elements between the C / D matrices of two batch entries (batched only)
  int32_t tiles_n;
  int32_t raster_band;
  int32_t out_kind;
  int32_t out_col_major;      // quantised outputs only: D is stored column-major (M contiguous, ldd = its pitch) and the
                              // scale factors cover 16 / 32 consecutive ROWS of a column: D^T with the K-major scale layout
  const __nv_bfloat16* C;
  void* D;
  uint8_t* SFD;
  int64_t ldc, ldd;           // elements
  float alpha, beta;
  const float* alpha_ptr;
  const float* beta_ptr;
  const float* norm_ptr;
  const float* alpha_array;   // grouped: one alpha per group (device), overrides alpha / alpha_ptr; or null
  const float* beta_array;
  const float* bias;          // fp32 vector added to alpha * acc before beta * C, or null
  int32_t bias_mode;          // 1: one entry per output column; 2: one per row of the (batched) problem
  int32_t bias_group_stride;  // mode 1: entries between the bias vectors of two groups (0: one vector for all)
  int32_t activation;         // kAct*: applied after alpha * acc + bias + beta * C, before the output conversion
  uint32_t* status;
  // Optional gating of A rows by flags (tensor-parallel all-gather): rows
  // [i*rows_per_flag, (i+1)*rows_per_flag) may be read once ready_flags[i] >= flag_target.
  const uint32_t* ready_flags;
  int32_t rows_per_flag;
  uint32_t flag_target;
  int32_t tile_m_rotate;      // dense only: start the M sweep at this tile row
  int32_t split_tail;         // 1: the tiles of the last wave of the persistent walk, when they fill at most half of the
                              // clusters, are computed as two halves of BN / 2 columns each, by twice as many clusters
                              // (BN == 256 only)
  int32_t debug_flags;        // only read when built with -DBSG_PROFILE (ablation switches, timeline capture)
  // Tensor-parallel all-gather of A (kernel template TP == true): the push warp of every CTA sends pieces of
  // this rank's row shard of A and SFA into every peer's gathered buffer.
  int32_t tp_world, tp_rank;
  int32_t tp_rows_per_shard;  // multiple of 256
  int32_t tp_ksplit;          // pieces a 256-row block is cut into (one flag increment each)
  int32_t tp_push_in_kernel;  // 1: the push warp moves the data; 0: the host's copy-engine transfers do
  int32_t tp_release_announce; // 1: a batch of announcements is preceded by a proxy fence and a system-scope release fence
  int32_t tp_paced_push;      // 2: as 1, and the pieces are spread over that stage; 1: the shard for the j-th nearest consumer is pushed while this CTA works on stage j - 1
                              //    of its own walk (all ranks walk in step, so it arrives one stage before it is needed),
                              //    instead of everything as fast as the links allow at the start of the kernel
  uint32_t tp_epoch;          // call counter, starts at 1; the peers use the same value
  uint32_t tp_ready_target;       // a peer's buffer may be filled once its "launched call" word has reached this
  int32_t tp_remote_row_offset;   // rows between the buffer this call gathers into and buffer 0 (0 or M)
  int64_t tp_row_bytes;       // bytes of one row of A
  int64_t tp_sfa_rowatom_bytes;   // bytes of one 128-row atom row of SFA (512 * k_atoms)
  // GEMM + reduce-scatter (kernel template RS == true): every rank multiplies its K shard for all M x N; the partial
  // sums of a slice of rows travel around the ring of ranks, one hop per stage, each hop adding its own partial, and
  // end at the rank that owns the slice.  The walk over the M tiles starts at slice rank + 1 (tile_m_rotate), so
  // stage s = walk position / rs_tiles_per_slice.  Stage 0 adds nothing; stages >= 1 add the partial received from
  // rank + 1; stages < world - 1 store into the receive buffer of rank - 1; the last stage stores the result.
  int32_t rs_world;
  int32_t rs_tiles_per_slice;     // M tiles per slice (rs_slice_rows / tile M)
  int32_t rs_slice_rows;
  int32_t rs_parity_rows;         // first row, in the receive buffers, of the half that this call uses (calls alternate)
  uint32_t rs_flag_target;        // arrivals a received tile must show: 4 * CG per call that used this half so far
  uint32_t rs_ready_target;       // the left neighbour's receive half is free once it has launched this call number
  uint32_t rs_epoch;
  const __nv_bfloat16* rs_recv;   // this rank's receive buffers: [2 halves][world - 1 stages][rs_slice_rows][N] bf16
  uint32_t* rs_flags;             // arrival counters of the tiles in rs_recv: [2][world - 1][rs_tiles_per_slice][tiles_n]
  uint32_t* rs_flags_left;        // the same array of rank - 1
  uint32_t* rs_sync;              // this rank's sync words: [0] = call number the right neighbour ... see kRsSync*
  uint32_t* rs_sync_left;         // sync words of rank - 1
  uint32_t* rs_sync_right;        // sync words of rank + 1
  // GEMM + all-reduce on top of the reduce-scatter: in the last stage the finished slice is stored into EVERY rank's
  // full-size output (M x N, two halves used by alternate calls) instead of this rank's D.
  int32_t rs_allreduce;
  int32_t rs_rank;
  int32_t rs_out_half;            // which half of the outputs this call writes
  uint32_t rs_done_target;        // this rank's arrival counter shows this once every peer's slice of this call is in place
  const CUtensorMap* rs_out_maps; // [world] maps of the ranks' outputs (N, M, 2 halves), in this rank's global memory
  uint32_t* rs_peer_sync[8];      // sync words of every rank: [8 + q] = call number rank q has launched, [16] = arrival counter
  const GroupDesc* group_desc;    // pointer-array grouped form: one record per group (device memory)
  const uint8_t* tp_peer_a[8];    // gathered A buffer of every rank that this call fills (own entry = source: local buffer 0)
  const uint8_t* tp_peer_sfa[8];
  uint32_t* tp_peer_sync[8];      // sync words of every rank: [0,8) "rank q has launched call n", [32, ...) row-block counters
};

constexpr int kRsSyncLaunched = 0;   // word 0 of a rank's reduce-scatter sync words: the call number its LEFT neighbour has launched
constexpr int kRsSyncLaunchedBy = 8; // words 8 .. 15: the call number every rank has launched (all-reduce)
constexpr int kRsSyncArrived = 16;   // word 16: finished sub-tiles of other ranks' slices stored into this rank's output (all-reduce)
constexpr int kTpSyncReady = 0;
constexpr int kTpSyncFlags = 32;
constexpr uint32_t kStTimeoutPeer = 64u;      // tensor parallel: a peer never published / finished

template <int KIND, int CG, int BN, bool TP = false>
struct Cfg {
  static_assert(KIND >= kKindNvfp4 && KIND <= kKindMxfp8Mxfp4, "kind");
  static_assert(CG == 1 || CG == 2, "cta group");
  static_assert(BN == 64 || BN == 128 || BN == 192 || BN == 256, "tile n");
  static constexpr int kCtaM = 128;                       // accumulator rows per CTA (= TMEM lanes)
  static constexpr int kTileM = kCtaM * CG;               // rows per MMA tile
  static constexpr int kRowBytes = 128;                   // bytes of K per row per k-tile (one 128B swizzle atom)
  static constexpr int kTileK = kind_packs_fp4(KIND) ? 256 : 128;   // elements of K per k-tile
  static constexpr int kMmaK = kind_packs_fp4(KIND) ? 64 : 32;      // elements of K per instruction (32 bytes)
  static constexpr int kSfVec = KIND == kKindNvfp4 ? 16 : 32;
  static constexpr int kKAtoms = kTileK / kSfVec / 4;               // 512-byte SF atoms (4 K-blocks each) along K per k-tile
  static constexpr int kBRowsCta = BN / CG;               // rows of B each CTA loads
  static constexpr int kABytes = kCtaM * kRowBytes;
  static constexpr int kBBytes = kBRowsCta * kRowBytes;
  static constexpr int kSfaBytes = kKAtoms * 512;
  // 128-row atoms of SFB that the columns of one tile touch.  Tiles of 64 or 192 columns start in the middle of an atom
  // every other time: the atoms are fetched whole and the MMA is pointed at the right columns of tensor memory (a
  // column holds 32 rows of the atom), as the reference does for these tile widths
  // (include/cutlass/gemm/collective/sm100_blockscaled_mma_warpspecialized.hpp:719-741).
  static constexpr int kSfbAtoms = (BN + 127) / 128;
  static constexpr int kSfbCols = 4 * kSfbAtoms;            // tensor-memory columns of SFB per k-atom
  static constexpr int kSfbBytes = kSfbAtoms * kKAtoms * 512;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  // Bytes a stage's loads report to its barrier.  The mixed kind's B arrives as packed e2m1 that the TMA engine spreads
  // over twice the space (16 values in 8 bytes, then 8 bytes of padding): the transaction counts the 8, not the 16.
  static constexpr int kStageTxBytes = kStageBytes - (KIND == kKindMxfp8Mxfp4 ? kBBytes / 2 : 0);
#ifdef BSG_PROFILE
  static constexpr int kDbgBytes = (512 + 1024 + 256) * 4;   // instrumented build: in-kernel timeline stamps
#else
  static constexpr int kDbgBytes = 0;
#endif
  static constexpr int kCtlBytes = 8192 + kDbgBytes;
  static constexpr int kEpiBytes = 4 * 4096;              // per epilogue warp: 32 rows x 128 bytes of bf16 output
  static constexpr int kSmemLimit = 232448;               // 227 KB
  static constexpr int kTpChunk = 8192;                   // tensor parallel: bytes per bulk copy of the A push
  static constexpr int kTpBufs = 4;                       // staging buffers (ring)
  static constexpr int kTpReadLag = 2;                    // stores whose shared-memory read may still be pending
  static constexpr int kTpLag = 6;                        // a piece is announced this many chunks after its last store
  static constexpr int kTpPend = 4;                       // pieces that may wait for their announcement
  static constexpr int kTpBytes = TP ? kTpBufs * kTpChunk : 0;
  static constexpr int kStagesRaw = (kSmemLimit - kCtlBytes - kEpiBytes - kTpBytes - 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kTpBytes + kCtlBytes + 1024;
  // TMEM columns: two accumulators (overlapping by 48 columns when BN == 256), then SFA (16), then SFB (32).
  // One set of scale-factor columns: a second set, used by alternate k-tiles so that a k-tile's copies need not
  // wait for the previous k-tile's MMAs, was measured for both kinds and gained nothing (the copies and the MMAs
  // of one issuing thread run strictly in order in the tensor pipe).
  static constexpr int kAccStride = BN == 256 ? 208 : BN;
  static constexpr int kAccBars = BN == 256 ? 1 : 2;
  static constexpr int kSfaCol = 464;
  static constexpr int kSfbCol = 480;
  static constexpr int kPairs = BN / 64;                  // the epilogue drains 64 columns at a time
  static constexpr int kReleasePair = BN == 256 ? 0 : kPairs - 1;   // pair after whose load the accumulator is released
};

constexpr int kSchedSlots = 4;

struct alignas(16) Ctl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t tp_full[8];      // tensor parallel: staging buffer filled
  // Dynamic scheduler: ring of kSchedSlots work ids.  sched_full[s] (every CTA): slot s holds the next work id;
  // sched_empty[s] (leader CTA): every consumer warp of the cluster has read it; clc_bar[s] (leader): the
  // answer of the cancellation request for slot s has landed in clc_response[s].
  uint64_t sched_full[4];
  uint64_t sched_empty[4];
  uint64_t clc_bar[4];
  alignas(16) uint32_t clc_response[4][4];
  int32_t sched_w[4];
  uint32_t tmem_base;
  volatile uint32_t abort;
  volatile int32_t tp_stage_now;   // tensor parallel: stage (shard index in consumption order) of the tile the producer is on
  volatile int32_t tp_progress;    // how far this CTA's producer is through its own work, in 1/1024 of a stage (all CTAs of all
                                   // ranks work through their items at the same rate, so this is also the time in stages)
  int32_t total_tiles;
  int32_t pad;
  int32_t tile_start[kMaxGroups + 1];
  int32_t row0[kMaxGroups];
  int32_t rows[kMaxGroups];
  int32_t atom0[kMaxGroups];
  int32_t gN[kMaxGroups];   // pointer-array grouped form: N and K of every group
  int32_t gK[kMaxGroups];
};
static_assert(sizeof(Ctl) <= 8192, "control block too large");

struct TileInfo {
  int32_t g, tm, tn;
  int32_t row0;       // first row of the tile in A / D
  int32_t row_end;    // end row of the group
  int32_t group_row0; // first row of the group
  int32_t sf_atom;    // SFA / SFD row-atom index of the tile's first row
  int32_t group_atom0;
  int32_t map_row0;   // row coordinate of the tile's first row in the A / D tensor maps
  int32_t map_l;      // third coordinate there (batch entry; 0 when rows run over all groups)
  int32_t tm_walk;    // position of the tile row in the walk over M (before the rotation of the starting row)
  int32_t N, K;       // extents of the tile's problem (those of its group in the pointer-array form)
};

// Group that holds tile t (binary search in the prefix of tile counts).
__device__ __forceinline__ int32_t group_of_tile(const Ctl* ctl, int32_t num_groups, int32_t t) {
  int lo = 0, hi = num_groups;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (ctl->tile_start[mid] <= t) lo = mid; else hi = mid;
  }
  return lo;
}

// `bn` / `ptr`: tile width and whether the groups have extents of their own (both compile-time at the call sites).
__device__ __forceinline__ TileInfo decode_tile(const Ctl* ctl, const GemmParams& p, int32_t t, int32_t tile_m, int32_t bn, bool ptr) {
  const int lo = group_of_tile(ctl, p.num_groups, t);
  TileInfo ti;
  ti.g = lo;
  ti.N = ptr ? ctl->gN[lo] : p.N;
  ti.K = ptr ? ctl->gK[lo] : p.K;
  const int32_t tiles_n = ptr ? (ti.N + bn - 1) / bn : p.tiles_n;
  const int32_t local = t - ctl->tile_start[lo];
  const int32_t rows = ctl->rows[lo];
  const int32_t tiles_m = (rows + tile_m - 1) / tile_m;
  const int32_t band = p.raster_band;
  const int32_t per_band = band * tiles_n;
  const int32_t b = local / per_band;
  const int32_t rem = local - b * per_band;
  const int32_t bh = min(band, tiles_m - b * band);
  int32_t tm = b * band + rem % bh;
  ti.tn = rem / bh;
  ti.tm_walk = tm;
  if (p.tile_m_rotate != 0) tm = (tm + p.tile_m_rotate) % tiles_m;
  ti.tm = tm;
  ti.group_row0 = ctl->row0[lo];
  ti.row0 = ti.group_row0 + tm * tile_m;
  ti.row_end = ti.group_row0 + rows;
  ti.group_atom0 = ctl->atom0[lo];
  ti.sf_atom = ti.group_atom0 + tm * (tile_m / 128);
  ti.map_row0 = p.batched ? tm * tile_m : ti.row0;
  ti.map_l = p.batched ? lo : 0;
  return ti;
}

// Slow path of a barrier wait; only reached when the fast spin gave up, i.e. when
// something is wrong or the machine is badly oversubscribed.  Bounded by SM cycles.
__device__ __noinline__ uint32_t slow_wait(uint32_t bar, uint32_t parity, Ctl* ctl) {
  const long long t0 = clock64();
  while (true) {
    if (ptx::mbar_spin(bar, parity, 64)) return 1;
    const long long limit = ctl->abort ? 40000ll : 4000000000ll;   // ~20 us once aborting, else ~2 s
    if (clock64() - t0 > limit) break;
  }
  ctl->abort = 1;
  return 0;
}

// Bounded wait on an mbarrier phase.  `dead` is this thread's sticky failure flag: once a wait
// has timed out, later waits give up quickly so that the kernel still terminates in bounded time.
__device__ __forceinline__ void wait_barrier(uint32_t bar, uint32_t parity, Ctl* ctl, uint32_t& dead) {
  uint32_t ok = ptx::mbar_spin(bar, parity, dead ? 16u : 100000u);
  if (!ok) {
    ok = dead ? 0u : slow_wait(bar, parity, ctl);
    if (!ok) dead = 1;
  }
}

__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart (SBO), LBO unused (1), descriptor version 1.
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t smem_addr) {
  // Un-swizzled K-major 32 rows x 16 bytes: 8-row groups 128 bytes apart.
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (8ull << 32) | (1ull << 46);
}

template <int KIND, int CG>
__device__ __forceinline__ constexpr uint32_t make_idesc(uint32_t n) {
  // Operand formats: the 4-bit kinds (mxf4nvf4, mxf4) number E2M1 as 1; kind::mxf8f6f4 numbers E4M3 as 0 and E2M1 as 5.
  constexpr uint32_t a_fmt = kind_packs_fp4(KIND) ? 1u : 0u;
  constexpr uint32_t b_fmt = kind_packs_fp4(KIND) ? 1u : (KIND == kKindMxfp8Mxfp4 ? 5u : 0u);
  constexpr uint32_t sf_fmt = KIND == kKindNvfp4 ? 0u : 1u;    // UE4M3 / UE8M0
  constexpr uint32_t m = 128u * CG;
  return (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (sf_fmt << 23) | ((m >> 4) << 24);
}

// Work item w of the persistent walk -> (tile, half): items below split_from are whole tiles; above it every tile
// appears twice, once per half of its columns.
struct WorkItem {
  int32_t t;       // tile index
  int32_t half;    // 0 or 1: which BN / 2 columns (split items only)
  bool split;
};
__device__ __forceinline__ WorkItem decode_work(int32_t w, int32_t split_from) {
  WorkItem wi;
  wi.split = w >= split_from;
  wi.t = wi.split ? split_from + ((w - split_from) >> 1) : w;
  wi.half = wi.split ? ((w - split_from) & 1) : 0;
  return wi;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ int32_t bcast(int32_t v) { return __shfl_sync(0xffffffffu, v, 0); }
__device__ __forceinline__ uint32_t bcast(uint32_t v) { return __shfl_sync(0xffffffffu, v, 0); }

__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded spin until *flag >= target (system-scope acquire).  Returns false on timeout.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t target, Ctl* ctl) {
  if (ptx::ld_acquire_sys_u32(flag) >= target) return true;
  const long long t0 = clock64();
  while (ptx::ld_acquire_sys_u32(flag) < target) {
    if (ctl->abort || clock64() - t0 > 4000000000ll) { ctl->abort = 1; return false; }
    __nanosleep(100);
  }
  return true;
}

// Walks the chunks that one CTA pushes in a tensor-parallel call: pieces c = cta, cta + grid, ...
// (a piece = 256 / ksplit rows of one 256-row block of this rank's shard for one destination rank;
// the first piece of a block also carries the block's two SFA row atoms); every piece is one or
// three contiguous spans, every span is cut into chunks of at most `chunk_bytes`.
struct TpChunkIter {
  int c, grid, total, per_shard, span, last_span, chunk_bytes;
  int dst_rank, row_block;
  int64_t span_off, span_bytes, done;
  uint32_t bytes;
  bool last_of_piece;
  __device__ __forceinline__ bool valid() const { return c < total; }
  __device__ __forceinline__ void load_piece(const GemmParams& p) {
    if (c >= total) return;
    const int j = c / per_shard + 1;
    dst_rank = (p.tp_rank - j + p.tp_world) % p.tp_world;     // rank-1 consumes this shard first
    span = 0;
    load_span(p);
  }
  __device__ __forceinline__ void load_span(const GemmParams& p) {
    const int j = c / per_shard + 1;
    const int rem = c - (j - 1) * per_shard;
    // The piece that also carries the scale factors (ks == 0) sits at a different place in every row
    // block, so that those larger pieces spread over the CTAs whatever the grid size.
    const int rb = rem / p.tp_ksplit, ks = (rem + rb) % p.tp_ksplit;
    const int64_t row0 = int64_t(p.tp_rank) * p.tp_rows_per_shard + int64_t(rb) * 256;
    row_block = int(row0 / 256);
    last_span = ks == 0 ? 2 : 0;     // the first piece of a row block also carries the block's scale factors
    if (span == 0) {
      const int rows = 256 / p.tp_ksplit;
      span_off = (row0 + int64_t(ks) * rows) * p.tp_row_bytes;
      span_bytes = int64_t(rows) * p.tp_row_bytes;
    } else {
      span_bytes = p.tp_sfa_rowatom_bytes;
      span_off = (row0 / 128 + (span - 1)) * p.tp_sfa_rowatom_bytes;
    }
    done = 0;
    set_chunk();
  }
  __device__ __forceinline__ void set_chunk() {
    const int64_t left = span_bytes - done;
    bytes = uint32_t(left < chunk_bytes ? left : chunk_bytes);
    last_of_piece = (span == last_span) && (done + bytes >= span_bytes);
  }
  __device__ __forceinline__ void init(const GemmParams& p, int cta, int grid_, int chunk_bytes_) {
    grid = grid_;
    chunk_bytes = chunk_bytes_;
    per_shard = (p.tp_rows_per_shard / 256) * p.tp_ksplit;
    total = (p.tp_world - 1) * per_shard;
    c = cta;
    load_piece(p);
  }
  __device__ __forceinline__ void next(const GemmParams& p) {
    done += bytes;
    if (done < span_bytes) { set_chunk(); return; }
    if (span < last_span) { ++span; load_span(p); return; }
    c += grid;
    load_piece(p);
  }
  __device__ __forceinline__ const uint8_t* src(const GemmParams& p) const {
    return (span == 0 ? p.tp_peer_a[p.tp_rank] : p.tp_peer_sfa[p.tp_rank]) + span_off + done;
  }
  __device__ __forceinline__ uint8_t* dst(const GemmParams& p) const {
    return const_cast<uint8_t*>(span == 0 ? p.tp_peer_a[dst_rank] : p.tp_peer_sfa[dst_rank]) + span_off + done;
  }
};

// Waits until all but the newest `n` bulk stores of this thread have read their shared-memory source.
__device__ __forceinline__ void tp_wait_read(uint32_t n) {
  if (n == 0u) ptx::bulk_wait_group_read<0>();
  else if (n == 1u) ptx::bulk_wait_group_read<1>();
  else if (n == 2u) ptx::bulk_wait_group_read<2>();
  else if (n == 4u) ptx::bulk_wait_group_read<4>();
  else ptx::bulk_wait_group_read<6>();
}

// Side-stream helpers of the copy-engine mode of the tensor-parallel GEMM.
// Waits (bounded) until every peer has launched call `epoch`, i.e. its gathered buffer may be overwritten.
__global__ void tp_wait_peers_kernel(const uint32_t* sync, int world, int rank, uint32_t epoch, uint32_t* status) {
  if (threadIdx.x != 0) return;
  const long long t0 = clock64();
  for (int q = 0; q < world; ++q) {
    if (q == rank) continue;
    while (ptx::ld_acquire_sys_u32(sync + kTpSyncReady + q) < epoch) {
      if (clock64() - t0 > 4000000000ll) { atomicOr(status, kStTimeoutPeer); return; }
      __nanosleep(200);
    }
  }
}
// Announces `blocks` row blocks (starting at `first`) as arrived in a peer's buffer: stream order puts
// this after the copy-engine transfers that filled them.
__global__ void tp_announce_kernel(uint32_t* peer_flags, int first, int blocks, uint32_t add) {
  const int i = threadIdx.x;
  if (i < blocks) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(peer_flags + first + i), "r"(add) : "memory");
  }
}

// Element-wise activations of the reference (include/cutlass/epilogue/thread/activation.h): ReLu :145 (max with 0),
// GELU<float> :585 ((0.5 x) (1 + erf(x / sqrt 2))), SiLu :452 (x * 1 / (1 + exp(-x))), same operation order.
__device__ __forceinline__ float apply_activation(float x, int act) {
  switch (act) {
    case kActRelu: return x != x ? x : fmaxf(x, 0.0f);
    case kActGelu: return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, erff(__fmul_rn(x, 0.70710678118654752440f))));
    case kActSilu: return __fmul_rn(x, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))));
    default: return x;
  }
}

// Consumer side of the dynamic scheduler's ring: step k of the walk -> the work id published for it (-1: no more
// work).  Called by a whole warp; lane 0 reports the slot as read to the leader CTA.
template <int CG>
__device__ __forceinline__ int32_t sched_consume(Ctl* ctl, uint32_t k, uint32_t& dead) {
  const uint32_t slot = k % kSchedSlots, phase = (k / kSchedSlots) & 1u;
  wait_barrier(ptx::smem_u32(&ctl->sched_full[slot]), phase, ctl, dead);
  asm volatile("fence.acq_rel.cluster;" ::: "memory");      // the id may have been written by the other CTA of the pair
  const int32_t w = *reinterpret_cast<volatile int32_t*>(&ctl->sched_w[slot]);
  __syncwarp();
  if ((threadIdx.x & 31) == 0) {
    const uint32_t bar = ptx::smem_u32(&ctl->sched_empty[slot]);
    if constexpr (CG == 2) ptx::mbar_arrive_remote(ptx::mapa(bar, 0));
    else ptx::mbar_arrive(bar);
  }
  return dead ? -1 : w;
}

// OUTX: the instantiations that also write fp16 / fp32 outputs and column-major quantised outputs.  They are separate
// because the extra epilogue branches, although never taken otherwise, were measured to cost the bf16 and the
// re-quantising epilogues 1 - 6 % (and the column-major path alone 38 registers per thread).
template <int KIND, int CG, int BN, bool TP = false, bool DYN = false, bool RS = false, bool PTR = false, bool OUTX = false>
__global__ void __launch_bounds__(TP ? 224 : 192, 1)
bsg_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmDpeer, const GemmParams p) {
  using C = Cfg<KIND, CG, BN, TP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + C::kStages * C::kABytes;
  uint8_t* sEpi = sB + C::kStages * C::kBBytes;                 // 1024-byte aligned (swizzled TMA-store source)
  uint8_t* sTp = sEpi + C::kEpiBytes;                           // tensor parallel: push staging (128-byte aligned)
  uint8_t* sSFA = sTp + C::kTpBytes;
  uint8_t* sSFB = sSFA + C::kStages * C::kSfaBytes;
  Ctl* ctl = reinterpret_cast<Ctl*>(sSFB + C::kStages * C::kSfbBytes);

  const int warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0);   // warp-uniform for the compiler
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = CG == 2 ? ptx::cluster_ctarank() : 0u;
  const bool is_leader = cta_rank == 0;
  const int32_t cluster_idx = CG == 2 ? int32_t(ptx::cluster_id_x()) : int32_t(blockIdx.x);
  const int32_t num_clusters = CG == 2 ? int32_t(ptx::num_clusters_x()) : int32_t(gridDim.x);

  // ------------------------------------------------------------------ setup
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->tmem_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->tmem_empty[s]), 4 * CG);
    }
    for (int s = 0; s < 8; ++s) ptx::mbar_init(ptx::smem_u32(&ctl->tp_full[s]), 1);
    for (int s = 0; s < kSchedSlots; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->sched_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->sched_empty[s]), 5 * CG);   // leader: MMA + 4 epilogue warps; other CTA: producer + 4
      ptx::mbar_init(ptx::smem_u32(&ctl->clc_bar[s]), 1);
    }
    ctl->abort = 0;
    ctl->tp_stage_now = 0;
    ctl->tp_progress = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async();
  }
  if (!PTR && warp == 5 && lane == 0) {
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
    ptx::prefetch_tmap(&tmSFA);
    ptx::prefetch_tmap(&tmSFB);
    ptx::prefetch_tmap(&tmD);
    if constexpr (RS) ptx::prefetch_tmap(&tmDpeer);
  }
  // Programmatic dependent launch: everything above overlaps the tail of the previous kernel on the stream; from
  // here on global memory is touched, which needs that kernel complete.  The kernel after this one may start its
  // own set-up as soon as SMs free up (it waits at the same place).  Both are no-ops in an ordinary launch.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  if constexpr (RS) {
    // Launching this call means the previous one has finished reading its receive buffers: tell rank + 1, which
    // stores into them, that the half of the call after this one may be overwritten.
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.rs_world > 1) {
      __threadfence_system();
      st_release_sys_u32(p.rs_sync_right + kRsSyncLaunched, p.rs_epoch);
      // All-reduce: every rank stores into this rank's output; its half of two calls ago has been read by now.
      if (p.rs_allreduce) {
        for (int q = 0; q < p.rs_world; ++q) {
          if (q != p.rs_rank) st_release_sys_u32(p.rs_peer_sync[q] + kRsSyncLaunchedBy + p.rs_rank, p.rs_epoch);
        }
      }
    }
  }
  // Group table: end rows first (parallel), then a serial prefix by one thread.
  for (int g = threadIdx.x; g < p.num_groups; g += blockDim.x) {
    if constexpr (PTR) {
      const GroupDesc* gd = p.group_desc + g;
      ctl->rows[g] = gd->M;
      ctl->gN[g] = gd->N;
      ctl->gK[g] = gd->K;
    } else {
      ctl->rows[g] = p.offsets ? p.offsets[g] : (g + 1) * p.rows_per_group;   // holds END rows for now
    }
  }
  __syncthreads();
  if (threadIdx.x == 32) {
    int32_t prev_end = 0, tiles = 0, atoms = 0;
    bool bad = false;
    for (int g = 0; g < p.num_groups; ++g) {
      if constexpr (PTR) {
        // every group starts at row 0 of its own tensors
        const int32_t rows = max(ctl->rows[g], 0);
        ctl->tile_start[g] = tiles;
        ctl->row0[g] = 0;
        ctl->rows[g] = rows;
        ctl->atom0[g] = 0;
        tiles += ((rows + C::kTileM - 1) / C::kTileM) * ((max(ctl->gN[g], 0) + BN - 1) / BN);
      } else {
        int32_t end = ctl->rows[g];
        if (end < prev_end || end > p.total_rows) { bad = true; end = prev_end; }
        const int32_t rows = end - prev_end;
        ctl->tile_start[g] = tiles;
        ctl->row0[g] = prev_end;
        ctl->rows[g] = rows;
        ctl->atom0[g] = atoms;
        tiles += ((rows + C::kTileM - 1) / C::kTileM) * p.tiles_n;
        atoms += (rows + 127) / 128;
        prev_end = end;
      }
    }
    ctl->tile_start[p.num_groups] = tiles;
    ctl->total_tiles = tiles;
    if (bad) atomicOr(p.status, kStBadOffsets);
  }
  if (warp == 4) {
    ptx::tmem_alloc<CG>(ptx::smem_u32(&ctl->tmem_base), 512);
    ptx::tmem_relinquish<CG>();
  }
  ptx::tc_fence_before();
  if constexpr (CG == 2) { ptx::cluster_arrive(); ptx::cluster_wait(); } else { __syncthreads(); }
  ptx::tc_fence_after();

  const uint32_t tmem_base = bcast(ctl->tmem_base);
  const int32_t total_tiles = bcast(ctl->total_tiles);
  // Tail of the walk: with T tiles on G clusters the last wave holds T mod G tiles; if that is at most G / 2 its tiles
  // are split (see split_tail), which shortens the last wave to half a tile time.
  int32_t split_from = total_tiles;
  if (BN == 256 && !DYN && !RS && p.split_tail != 0 && total_tiles > num_clusters) {
    const int32_t tail = total_tiles % num_clusters;
    if (tail > 0 && 2 * tail <= num_clusters) split_from = total_tiles - tail;
  }
  const int32_t total_work = split_from + 2 * (total_tiles - split_from);
  // Walk of the work items.  Static: cluster c takes items c, c + G, c + 2G, ...  Dynamic: one cluster per work item
  // was launched; a running cluster starts with its own id and, after each item, takes over the id of a cluster that
  // has not started yet by cancelling it (work ids beyond total_work are skipped: the launch only knows an upper bound
  // when the group sizes live on the device).  -1 ends the walk.
  const int32_t first_work = (DYN || cluster_idx < total_work) ? cluster_idx : -1;
  auto static_next = [&](int32_t w) { w += num_clusters; return w < total_work ? w : -1; };
  const int32_t k_tiles = (p.K + C::kTileK - 1) / C::kTileK;
  uint32_t dead = 0;
#ifdef BSG_PROFILE
  // Timeline capture (instrumented build only, debug_flags != 0): the first cluster's leader CTA collects stamps
  // (code << 26 | low 26 bits of the SM clock) in shared memory, regions of 512 / 1024 / 256 entries for the
  // producer, MMA and epilogue warps (entry 0 = count), and copies them behind the first 1024 bytes of the
  // workspace when the kernel ends.
  uint32_t* dbg_s = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(ctl) + 8192);
  const bool dbg_on = p.debug_flags != 0 && cluster_idx == 0 && is_leader;
  uint32_t dbg_n = 1;
#define BSG_DBG(region, code) do { if (dbg_on && lane == 0) { constexpr int o_ = (region) == 0 ? 0 : (region) == 1 ? 512 : 1536; \
    constexpr int cap_ = (region) == 0 ? 512 : (region) == 1 ? 1024 : 256; \
    if (dbg_n < cap_) { dbg_s[o_ + dbg_n++] = (uint32_t(code) << 26) | (uint32_t(clock64()) & 0x3FFFFFFu); dbg_s[o_] = dbg_n; } } } while (0)
  if (dbg_on && threadIdx.x < 3) dbg_s[threadIdx.x == 0 ? 0 : threadIdx.x == 1 ? 512 : 1536] = 1;
#else
#define BSG_DBG(region, code) do { } while (0)
#endif

  if (warp == 5) {
    // ---------------------------------------------------------------- TMA producer
    const uint32_t elected = ptx::elect_one_sync();
    const uint32_t sA0 = ptx::smem_u32(sA), sB0 = ptx::smem_u32(sB);
    const uint32_t sSFA0 = ptx::smem_u32(sSFA), sSFB0 = ptx::smem_u32(sSFB);
    const uint32_t full0 = ptx::smem_u32(&ctl->full[0]), empty0 = ptx::smem_u32(&ctl->empty[0]);
    const uint32_t full0_leader = CG == 2 ? ptx::mapa(full0, 0) : full0;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t step = 0;
    // work items of this cluster in the static walk (tensor parallel: the measure of its progress)
    const int32_t tp_own_items = max(1, (total_work - cluster_idx + num_clusters - 1) / num_clusters);
    for (int32_t w = first_work; w >= 0; ++step) {
      if constexpr (DYN) {
        if (is_leader) {
          // Ask for the work item after this one now; the answer is read once this item's loads are issued.
          const uint32_t slot = step % kSchedSlots, sphase = (step / kSchedSlots) & 1u;
          wait_barrier(ptx::smem_u32(&ctl->sched_empty[slot]), sphase ^ 1u, ctl, dead);
          if (elected && !dead) {
            const uint32_t bar = ptx::smem_u32(&ctl->clc_bar[slot]);
            ptx::mbar_arrive_expect_tx(bar, 16);
            ptx::clc_try_cancel(ptx::smem_u32(&ctl->clc_response[slot][0]), bar);
          }
        }
      }
      if (w < total_work) {
      const WorkItem wi = decode_work(w, split_from);
      const TileInfo ti = decode_tile(ctl, p, wi.t, C::kTileM, BN, PTR);
      // Tensor parallel: rows of other ranks are read from the gathered buffer of this call, which lies
      // tp_remote_row_offset rows behind buffer 0 in the same tensor map; own rows always from buffer 0.
      if constexpr (TP) {
        if (lane == 0) ctl->tp_stage_now = ti.tm_walk / (p.tp_rows_per_shard / C::kTileM);
      }
      const bool tp_remote = TP && ti.row0 / p.tp_rows_per_shard != p.tp_rank;
      const int32_t tp_row_off = tp_remote ? p.tp_remote_row_offset : 0;
      const int32_t a_row = bcast(ti.map_row0 + int32_t(cta_rank) * C::kCtaM + tp_row_off);
      const int32_t a_l = bcast(ti.map_l);
      // A half tile needs BN / 4 rows of B per CTA; the box still brings kBRowsCta rows, of which the MMA reads the first.
      const int32_t b_row = bcast(ti.tn * BN + (wi.split ? wi.half * (BN / 2) + int32_t(cta_rank) * (C::kBRowsCta / 2)
                                                         : int32_t(cta_rank) * C::kBRowsCta));
      const int32_t b_l = bcast(p.b_per_group ? ti.g : 0);
      // The second CTA of a pair may lie wholly past the group's last row: keep its
      // scale-factor fetch inside the group's own atoms (its rows are never stored).
      const int32_t group_atoms = (ti.row_end - ti.group_row0 + 127) >> 7;
      const int32_t sfa_atom = bcast(min(ti.sf_atom + int32_t(cta_rank), ti.group_atom0 + max(group_atoms, 1) - 1) + (tp_row_off >> 7));
      const int32_t sfb_atom = bcast(ti.g * p.sfb_atoms_per_group + (ti.tn * BN) / 128 + wi.half);
      // Pointer-array form: the group's own tensor maps (in global memory) and depth.
      const CUtensorMap *mapA = &tmA, *mapB = &tmB, *mapSFA = &tmSFA, *mapSFB = &tmSFB;
      int32_t tile_k_tiles = k_tiles;
      if constexpr (PTR) {
        const GroupDesc* gd = p.group_desc + bcast(ti.g);
        mapA = &gd->tmA; mapB = &gd->tmB; mapSFA = &gd->tmSFA; mapSFB = &gd->tmSFB;
        tile_k_tiles = bcast((ti.K + C::kTileK - 1) / C::kTileK);
        if (elected) {
          ptx::fence_tensormap_acquire(mapA); ptx::fence_tensormap_acquire(mapB);
          ptx::fence_tensormap_acquire(mapSFA); ptx::fence_tensormap_acquire(mapSFB);
        }
      }
      if (p.ready_flags != nullptr && (!TP || tp_remote)) {
        const uint32_t* flag = p.ready_flags + ti.row0 / p.rows_per_flag;
        const long long t0 = clock64();
        while (ptx::ld_acquire_sys_u32(flag) < p.flag_target) {
          if (dead || ctl->abort || clock64() - t0 > 4000000000ll) {
            if (!dead) atomicOr(p.status, kStTimeoutFlag);
            dead = 1;
            ctl->abort = 1;
            break;
          }
          __nanosleep(64);
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        __syncwarp();
      }
      for (int32_t kt = 0; kt < tile_k_tiles; ++kt) {
        if constexpr (TP) {
          if (p.tp_paced_push == 2 && lane == 0 && (kt & 7) == 0)
            ctl->tp_progress = int32_t((int64_t(step) * tile_k_tiles + kt) * 1024 * p.tp_world / (int64_t(tp_own_items) * tile_k_tiles));
        }
        wait_barrier(empty0 + stage * 8, phase ^ 1u, ctl, dead);
        BSG_DBG(0, 1);
        // After a timeout nothing more is issued: free-running loads would overrun the barriers' byte counts.
        if (elected && !dead) {
          const uint32_t full_local = full0 + stage * 8;
          if (is_leader) ptx::mbar_arrive_expect_tx(full_local, uint32_t(C::kStageTxBytes) * CG);
          const uint32_t bar = full0_leader + stage * 8;
          ptx::tma_load_3d<CG>(sA0 + stage * C::kABytes, mapA, bar, kt * C::kRowBytes, a_row, a_l);
          ptx::tma_load_3d<CG>(sB0 + stage * C::kBBytes, mapB, bar, kt * C::kRowBytes, b_row, b_l);
          ptx::tma_load_3d<CG>(sSFA0 + stage * C::kSfaBytes, mapSFA, bar, 0, kt * C::kKAtoms, sfa_atom);
          ptx::tma_load_3d<CG>(sSFB0 + stage * C::kSfbBytes, mapSFB, bar, 0, kt * C::kKAtoms, sfb_atom);
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
      }
      if constexpr (DYN) {
        if (is_leader) {
          // Publish the next work id to every consumer warp of the cluster.
          const uint32_t slot = step % kSchedSlots, sphase = (step / kSchedSlots) & 1u;
          wait_barrier(ptx::smem_u32(&ctl->clc_bar[slot]), sphase, ctl, dead);
          int32_t next = -1;
          if (!dead) {
            const uint32_t first_cta = ptx::clc_query_first_ctaid_x(ptx::smem_u32(&ctl->clc_response[slot][0]));
            next = first_cta == 0xFFFFFFFFu ? -1 : int32_t(first_cta / CG);
          }
          ptx::fence_proxy_async();      // the slot's next request overwrites the answer just read
          __syncwarp();
          if (lane == 0) {
            const uint32_t wslot = ptx::smem_u32(&ctl->sched_w[slot]);
            const uint32_t fbar = ptx::smem_u32(&ctl->sched_full[slot]);
            ctl->sched_w[slot] = next;
            ptx::mbar_arrive(fbar);
            if constexpr (CG == 2) {
              ptx::st_shared_cluster_u32(ptx::mapa(wslot, 1), uint32_t(next));
              ptx::mbar_arrive_remote(ptx::mapa(fbar, 1));
            }
          }
          w = next;
        } else {
          w = sched_consume<CG>(ctl, step, dead);
        }
      } else {
        w = static_next(w);
      }
    }
    if constexpr (TP) {
      if (lane == 0) { ctl->tp_stage_now = 1 << 20; ctl->tp_progress = 1 << 30; }     // nothing left to pace against
    }
    // Tail: every stage must have been released, so that no commit-arrive is still
    // in flight towards this CTA's shared memory when it exits.
    for (int s = 0; s < C::kStages; ++s) {
      wait_barrier(empty0 + stage * 8, phase ^ 1u, ctl, dead);
      if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
    }
    if (dead) atomicOr(p.status, kStTimeoutEmpty);
  } else if (warp == 4) {
    // ---------------------------------------------------------------- UMMA issue
    if (is_leader) {
      constexpr uint32_t idesc_full = make_idesc<KIND, CG>(BN), idesc_half = make_idesc<KIND, CG>(BN / 2);
      const uint32_t elected = ptx::elect_one_sync();
      const uint32_t sA0 = ptx::smem_u32(sA), sB0 = ptx::smem_u32(sB);
      const uint32_t sSFA0 = ptx::smem_u32(sSFA), sSFB0 = ptx::smem_u32(sSFB);
      const uint32_t full0 = ptx::smem_u32(&ctl->full[0]), empty0 = ptx::smem_u32(&ctl->empty[0]);
      const uint32_t tfull0 = ptx::smem_u32(&ctl->tmem_full[0]), tempty0 = ptx::smem_u32(&ctl->tmem_empty[0]);
      int stage = 0;
      uint32_t phase = 0;
      int32_t it = 0;
      // `ready` holds the result of a non-blocking look at the NEXT stage's barrier, taken before the
      // current stage's instructions are issued, so that the barrier round trip overlaps the issue.
      uint32_t ready = 0;
      uint32_t step = 0;
      for (int32_t w = first_work; w >= 0; w = DYN ? sched_consume<CG>(ctl, step++, dead) : static_next(w)) {
        if (w >= total_work) continue;
        const uint32_t idesc = w >= split_from ? idesc_half : idesc_full;    // a half tile: the same operands, N = BN / 2
        const int acc_bar = it % C::kAccBars;
        const uint32_t acc_phase = uint32_t(it / C::kAccBars) & 1u;
        const uint32_t d_tmem = tmem_base + uint32_t(it & 1) * C::kAccStride;
        // tiles of 64 / 192 columns: the tile's first column inside its first SFB atom, in 32-row columns of tensor memory
        uint32_t sfb_off = 0;
        if constexpr (BN == 64 || BN == 192) {
          const TileInfo mti = decode_tile(ctl, p, decode_work(w, split_from).t, C::kTileM, BN, PTR);
          sfb_off = uint32_t(bcast(((mti.tn * BN) & 127) >> 5));
        }
        int32_t tile_K = p.K, tile_k_tiles = k_tiles;
        if constexpr (PTR) {
          tile_K = bcast(ctl->gK[group_of_tile(ctl, p.num_groups, decode_work(w, split_from).t)]);
          tile_k_tiles = (tile_K + C::kTileK - 1) / C::kTileK;
        }
        BSG_DBG(1, 9);
        wait_barrier(tempty0 + acc_bar * 8, acc_phase ^ 1u, ctl, dead);
        BSG_DBG(1, 10);
        ptx::tc_fence_after();
        for (int32_t kt = 0; kt < tile_k_tiles; ++kt) {
          if (!ready) wait_barrier(full0 + stage * 8, phase, ctl, dead);
          BSG_DBG(1, 11);
          int next_stage = stage + 1;
          uint32_t next_phase = phase;
          if (next_stage == C::kStages) { next_stage = 0; next_phase ^= 1u; }
          ready = ptx::mbar_spin_test(full0 + next_stage * 8, next_phase, 1);
          ptx::tc_fence_after();
          const uint32_t sfa_s = sSFA0 + stage * C::kSfaBytes;
          const uint32_t sfb_s = sSFB0 + stage * C::kSfbBytes;
          const uint64_t a_desc = make_desc_sw128(sA0 + stage * C::kABytes);
          const uint64_t b_desc = make_desc_sw128(sB0 + stage * C::kBBytes);
          const int32_t k_left = tile_K - kt * C::kTileK;
          const int n_mma = k_left >= C::kTileK ? 4 : (k_left + C::kMmaK - 1) / C::kMmaK;
          const uint32_t acc_flag = kt > 0 ? 1u : 0u;
          const uint32_t sfa_col = tmem_base + C::kSfaCol;
          const uint32_t sfb_col = tmem_base + C::kSfbCol;
          if (elected && !dead) {     // after a timeout no further tensor-core work or barrier arrival is issued
#pragma unroll
            for (int ka = 0; ka < C::kKAtoms; ++ka) {
              ptx::utccp_32x128b_warpx4<CG>(sfa_col + 4 * ka, make_desc_sf(sfa_s + ka * 512));
            }
#pragma unroll
            for (int ra = 0; ra < C::kSfbAtoms; ++ra) {
#pragma unroll
              for (int ka = 0; ka < C::kKAtoms; ++ka) {
                ptx::utccp_32x128b_warpx4<CG>(sfb_col + C::kSfbCols * ka + 4 * ra,
                                              make_desc_sf(sfb_s + (ra * C::kKAtoms + ka) * 512));
              }
            }
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
              if (kb < n_mma) {
                uint32_t sfa_t, sfb_t, id = idesc;
                if constexpr (KIND == kKindNvfp4) {
                  sfa_t = sfa_col + 4 * kb;                            // four scale factors per instruction: a column group each
                  sfb_t = sfb_col + C::kSfbCols * kb + sfb_off;
                } else if constexpr (KIND == kKindMxfp4) {
                  sfa_t = sfa_col + 4 * (kb >> 1);                     // two scale factors per instruction: half a column group
                  sfb_t = sfb_col + C::kSfbCols * (kb >> 1) + sfb_off;
                  id |= (uint32_t(kb & 1) << 5) | (uint32_t(kb & 1) << 30);   // lower / upper pair of the group's four bytes
                } else {
                  sfa_t = sfa_col;
                  sfb_t = sfb_col + sfb_off;
                  id |= (uint32_t(kb) << 4) | (uint32_t(kb) << 29);   // scale-factor byte of this K block
                }
                ptx::umma_block_scaled<KIND, CG>(d_tmem, a_desc + 2 * kb, b_desc + 2 * kb, id, sfa_t, sfb_t,
                                                 kb > 0 ? 1u : acc_flag);
              }
            }
            ptx::umma_commit<CG>(empty0 + stage * 8);
          }
          BSG_DBG(1, 12);
          stage = next_stage;
          phase = next_phase;
        }
        if (elected && !dead) ptx::umma_commit<CG>(tfull0 + acc_bar * 8);
        ++it;
      }
      if (dead) atomicOr(p.status, kStTimeoutFull | kStTimeoutTmemEmpty);
    }
  } else if (TP && warp == 6) {
    // ---------------------------------------------------------------- all-gather push warp (6)
    // This rank's own rows of A / SFA go into every peer's full-size buffer, nearest consumer first.
    // The data moves through the bulk-copy engine (global -> shared -> peer global) in chunks, with
    // kTpBufs chunks in flight; one elected lane issues everything.  Each finished piece bumps the
    // row-block counter in the peer's memory that the peer's TMA producer waits on.
    if (p.tp_world > 1) {
      const uint32_t elected = ptx::elect_one_sync();
      uint32_t* sync = p.tp_peer_sync[p.tp_rank];
      const uint32_t buf0 = ptx::smem_u32(sTp);
      const uint32_t bar0 = ptx::smem_u32(&ctl->tp_full[0]);
      bool peer_ok = true;
      // Launching this call means the previous one has finished reading its gathered buffer: tell every
      // peer, which may then fill that buffer again (with the data of the call after this one).
      if (blockIdx.x == 0 && elected) {
        __threadfence_system();
        for (int q = 0; q < p.tp_world; ++q) {
          if (q != p.tp_rank) st_release_sys_u32(p.tp_peer_sync[q] + kTpSyncReady + p.tp_rank, p.tp_epoch);
        }
      }
      TpChunkIter ld_it, st_it;                 // the load iterator runs ahead of the store iterator
      if (p.tp_push_in_kernel) {
      constexpr uint32_t nb = C::kTpBufs, ch = C::kTpChunk, rlag = C::kTpReadLag;
      ld_it.init(p, int(blockIdx.x), int(gridDim.x), int(ch));
      st_it.init(p, int(blockIdx.x), int(gridDim.x), int(ch));
      uint32_t n_ld = 0, n_st = 0;
      for (; n_ld < nb && ld_it.valid(); ++n_ld, ld_it.next(p)) {
        if (elected) {
          ptx::mbar_arrive_expect_tx(bar0 + n_ld * 8, ld_it.bytes);
          ptx::bulk_load(buf0 + n_ld * ch, ld_it.src(p), ld_it.bytes, bar0 + n_ld * 8);
        }
      }
      int checked = -1, paced_piece = -1;
      // Ring of staging buffers: chunk n goes through buffer n % nb.  A buffer is refilled `rlag` stores
      // after its own store was issued (by then that store has read it), so neither the load latency nor
      // the store's read latency is waited for in line.  A finished piece is announced kTpLag chunks
      // later, once its stores are known to be complete; up to kTpPend pieces wait in pend_*.
      int pend_rank[C::kTpPend], pend_block[C::kTpPend];
      uint32_t pend_due[C::kTpPend];
      int pend_head = 0, pend_cnt = 0;
      // The announcement is a system-scope add issued after wait_group has reported the piece's stores complete.
      // tp_release_announce (the library's default) puts a proxy fence and a system-scope release fence in front of
      // every batch of due announcements: the order the PTX memory model asks for between an async-proxy write and a
      // later generic-proxy write of the same thread.  Without it the add is relaxed and only the way bulk stores
      // complete over NVLink keeps it behind the data: faster (the fence also waits for the newer stores in flight),
      // but on eight GPUs a run of many small calls had a rank read a row block before its rows had landed.
      auto release_fences = [&]() {
        if (p.tp_release_announce) {
          asm volatile("fence.proxy.async;" ::: "memory");
          asm volatile("fence.acq_rel.sys;" ::: "memory");
        }
      };
      auto announce_head = [&]() {
        uint32_t* flag = p.tp_peer_sync[pend_rank[pend_head]] + kTpSyncFlags + pend_block[pend_head];
        asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(flag), "r"(1u) : "memory");
        pend_head = (pend_head + 1) % C::kTpPend;
        --pend_cnt;
      };
      // Before the warp sits down at a closed gate it announces what it has stored so far: a consumer may be waiting
      // for exactly those pieces, and the gate may only open once that consumer's rank has moved on in turn.
      auto flush_pending = [&]() {
        if (elected && pend_cnt > 0) {
          ptx::bulk_wait_group<0>();
          release_fences();
          while (pend_cnt > 0) announce_head();
        }
        __syncwarp();
      };
      for (; st_it.valid(); st_it.next(p), ++n_st) {
        const uint32_t b = n_st % nb;
        if (p.tp_paced_push == 2 && st_it.c != paced_piece) {
          // Spread push: the pieces for the j-th nearest consumer leave evenly over the first three quarters of
          // stage j - 1 of this CTA's walk (piece `rem` of the shard's `per_shard` at that fraction), so that the links
          // carry a steady flow instead of one burst per stage.
          const int j = st_it.c / st_it.per_shard + 1;
          const int rem = st_it.c - (j - 1) * st_it.per_shard;
          const int need = (j - 1) * 1024 + 768 * rem / st_it.per_shard;
          // A CTA whose tile is already at stage s counts as that far whatever its own pace (in a small problem a CTA
          // may start at a late stage and stand still there, waiting for rows that the peers send by the same rule).
          auto closed = [&]() { return max(ctl->tp_progress, min(ctl->tp_stage_now, 1 << 10) * 1024) < need; };
          if (bcast(int32_t(closed())) != 0) {       // one lane's look decides for the warp (flush_pending synchronises it)
            flush_pending();
            const long long t0 = clock64();
            while (closed() && !ctl->abort && clock64() - t0 < 4000000000ll) __nanosleep(200);
          }
          paced_piece = st_it.c;
        }
        if (st_it.dst_rank != checked) {
          if (p.tp_paced_push == 1) {
            // j-th nearest consumer: its rows are due when it starts stage j, which is when this rank does too
            const int j = (p.tp_rank - st_it.dst_rank + p.tp_world) % p.tp_world;
            if (bcast(int32_t(ctl->tp_stage_now < j - 1)) != 0) {
              flush_pending();
              const long long t0 = clock64();
              while (ctl->tp_stage_now < j - 1 && !ctl->abort && clock64() - t0 < 4000000000ll) __nanosleep(500);
            }
          }
          // The peer's buffer is free once the peer has launched the call after the one that last read it.
          if (!wait_flag_ge(sync + kTpSyncReady + st_it.dst_rank, p.tp_ready_target, ctl)) peer_ok = false;
          checked = st_it.dst_rank;
        }
        wait_barrier(bar0 + b * 8, (n_st / nb) & 1u, ctl, dead);
        if (dead) break;             // a staging load never landed: push and announce nothing more
        const bool refill = n_st >= rlag && ld_it.valid();
        if (elected) {
          if (pend_cnt > 0 && n_st >= pend_due[pend_head]) {
            ptx::bulk_wait_group<C::kTpLag>();
            release_fences();
            while (pend_cnt > 0 && n_st >= pend_due[pend_head]) announce_head();
          }
          if (peer_ok) ptx::bulk_store(st_it.dst(p), buf0 + b * ch, st_it.bytes);
          ptx::bulk_commit_group();
          if (st_it.last_of_piece && peer_ok) {
            if (pend_cnt == C::kTpPend) {
              ptx::bulk_wait_group<1>();   // everything but the store just issued
              release_fences();
              announce_head();
            }
            const int slot = (pend_head + pend_cnt) % C::kTpPend;
            pend_rank[slot] = st_it.dst_rank;
            pend_block[slot] = st_it.row_block;
            pend_due[slot] = n_st + 1 + C::kTpLag;    // by then at most kTpLag newer groups are outstanding
            ++pend_cnt;
          }
          if (refill) {
            tp_wait_read(rlag);      // the store issued `rlag` chunks ago has read its buffer
            const uint32_t rb = (n_st - rlag) % nb;
            ptx::mbar_arrive_expect_tx(bar0 + rb * 8, ld_it.bytes);
            ptx::bulk_load(buf0 + rb * ch, ld_it.src(p), ld_it.bytes, bar0 + rb * 8);
          }
        }
        if (refill) ld_it.next(p);
        __syncwarp();
      }
      if (elected && pend_cnt > 0) {
        ptx::bulk_wait_group<0>();
        release_fences();
        while (pend_cnt > 0) announce_head();
      }
      if (elected) ptx::bulk_wait_group<0>();
      }
      if (!peer_ok || dead) atomicOr(p.status, kStTimeoutPeer);
    }
  } else if (warp < 4) {
    // ---------------------------------------------------------------- epilogue (warps 0-3)
    const float alpha_all = p.alpha_ptr ? *p.alpha_ptr : p.alpha;
    const float beta_all = p.beta_ptr ? *p.beta_ptr : p.beta;
    float st = 0.f, st_scaled = 0.f;
    if (OUTX ? out_is_quantised(p.out_kind) : p.out_kind != kOutBf16) {
      st = p.norm_ptr ? *p.norm_ptr : 1.0f;
      st_scaled = __fmul_rn(st, __fdiv_rn(1.0f, p.out_kind == kOutNvfp4 ? 6.0f : 448.0f));
    }
    const int32_t sfd_vec = p.out_kind == kOutMxfp8 ? 32 : 16;
    const uint32_t tfull0 = ptx::smem_u32(&ctl->tmem_full[0]);
    const uint32_t tempty0 = ptx::smem_u32(&ctl->tmem_empty[0]);
    uint8_t* stage_buf = sEpi + warp * 4096;                     // this warp's 32 x 128-byte staging tile
    uint32_t n_store = 0;                                        // TMA stores issued so far (staging rotation)
    bool ar_ready = false;                                       // all-reduce: the peers' outputs may be written (checked once)
    int32_t it = 0;
    uint32_t step = 0;
    for (int32_t w = first_work; w >= 0; w = DYN ? sched_consume<CG>(ctl, step++, dead) : static_next(w)) {
      if (w >= total_work) continue;
      const WorkItem wi = decode_work(w, split_from);
      const TileInfo ti = decode_tile(ctl, p, wi.t, C::kTileM, BN, PTR);
      const int32_t tile_col0 = ti.tn * BN + wi.half * (BN / 2);       // first output column of this work item
      const int n_pairs = wi.split ? C::kPairs / 2 : C::kPairs;          // a half tile fills the accumulator's first BN / 2 columns
      // One alpha / beta per group when the arrays are given (grouped GEMM), else the scalars.
      const float alpha = p.alpha_array ? __ldg(p.alpha_array + ti.g) : alpha_all;
      const float beta = p.beta_array ? __ldg(p.beta_array + ti.g) : beta_all;
      // The problem this tile belongs to: the call's, or (pointer-array form) its group's own tensors and extents.
      const __nv_bfloat16* Cg = p.C;
      uint8_t* Dg = reinterpret_cast<uint8_t*>(p.D);
      uint8_t* SFDg = p.SFD;
      int64_t ldc = p.ldc, ldd = p.ldd;
      const CUtensorMap* mapD = &tmD;
      if constexpr (PTR) {
        const GroupDesc* gd = p.group_desc + ti.g;
        Cg = gd->C; Dg = reinterpret_cast<uint8_t*>(gd->D); SFDg = gd->SFD; ldc = gd->ldc; ldd = gd->ldd;
        mapD = &gd->tmD;
        if (lane == 0) ptx::fence_tensormap_acquire(mapD);
      }
      const int32_t prob_N = ti.N;
      const int32_t sfd_k_atoms = ((prob_N + sfd_vec - 1) / sfd_vec + 3) / 4;
      bool use_c = (Cg != nullptr) && (beta != 0.0f);
      // Reduce-scatter: stage of this tile row, where its addend comes from and where its result goes.
      int32_t rs_stage = 0;
      bool rs_to_peer = false;
      uint32_t* rs_flag_out = nullptr;
      if constexpr (RS) {
        rs_stage = ti.tm_walk / p.rs_tiles_per_slice;
        rs_to_peer = rs_stage < p.rs_world - 1;
        const int32_t tm_in_slice = ti.tm_walk - rs_stage * p.rs_tiles_per_slice;
        const int32_t half = p.rs_parity_rows != 0 ? 1 : 0;
        if (rs_stage >= 1) {
          // the partial sums of this tile from rank + 1: wait (bounded) until all of its warps have announced their stores
          const uint32_t* flag = p.rs_flags + ((int64_t(half) * (p.rs_world - 1) + (rs_stage - 1)) * p.rs_tiles_per_slice + tm_in_slice) * p.tiles_n + ti.tn;
          if (lane == 0 && !wait_flag_ge(flag, p.rs_flag_target, ctl)) dead = 1;
          dead = __shfl_sync(0xffffffffu, dead, 0);
          use_c = true;
        } else {
          use_c = false;
        }
        if (!rs_to_peer && p.rs_allreduce && !ar_ready) {
          // the finished slice goes to every rank: each must have launched this call (its output half is free then)
          if (lane == 0) {
            for (int q = 0; q < p.rs_world; ++q) {
              if (q != p.rs_rank && !wait_flag_ge(p.rs_sync + kRsSyncLaunchedBy + q, p.rs_epoch, ctl)) dead = 1;
              ptx::fence_tensormap_acquire(p.rs_out_maps + q);
            }
          }
          dead = __shfl_sync(0xffffffffu, dead, 0);
          ar_ready = true;
        }
        if (rs_to_peer) {
          rs_flag_out = p.rs_flags_left + ((int64_t(half) * (p.rs_world - 1) + rs_stage) * p.rs_tiles_per_slice + tm_in_slice) * p.tiles_n + ti.tn;
          // the neighbour's receive half is free once it has launched the call before the one that reads it again
          if (lane == 0 && !wait_flag_ge(p.rs_sync + kRsSyncLaunched, p.rs_ready_target, ctl)) dead = 1;
          dead = __shfl_sync(0xffffffffu, dead, 0);
        }
      }
      const int acc_bar = it % C::kAccBars;
      const uint32_t acc_phase = uint32_t(it / C::kAccBars) & 1u;
      const uint32_t acc_col = uint32_t(it & 1) * C::kAccStride;
      // While the mainloop of this tile still runs, the warp asks for its rows of C to be brought into L2 (a lane reads
      // 128 bytes of one row per 64 columns: without this every pair of the epilogue pays a DRAM round trip in line).
      const uint8_t* c_lane_row = nullptr;
      if (!RS && use_c) {
        const int32_t r_in_tile = int32_t(cta_rank) * C::kCtaM + warp * 32 + lane;
        if (ti.row0 + r_in_tile < ti.row_end) {
          c_lane_row = reinterpret_cast<const uint8_t*>(Cg + int64_t(ti.map_l) * p.batch_stride_c + int64_t(ti.map_row0 + r_in_tile) * ldc + tile_col0);
          const int32_t row_bytes = min(n_pairs * 128, (prob_N - tile_col0) * 2);
          for (int32_t o = 0; o < row_bytes; o += 128) ptx::prefetch_l2(c_lane_row + o);
          if (row_bytes > 0) ptx::prefetch_l2(c_lane_row + row_bytes - 1);       // a row need not start on a line boundary
        }
      }
      if (warp == 0) BSG_DBG(2, 19);
      wait_barrier(tfull0 + acc_bar * 8, acc_phase, ctl, dead);
      if (warp == 0) BSG_DBG(2, 20);
      __syncwarp();
      ptx::tc_fence_after();

      const int32_t cta_row0 = ti.row0 + int32_t(cta_rank) * C::kCtaM;
      const int32_t grow = cta_row0 + warp * 32 + lane;          // row over all groups
      const bool row_ok = grow < ti.row_end;
      const int32_t lrow = grow - ti.group_row0;                 // row within the group
      const int32_t warp_map_row0 = ti.map_row0 + int32_t(cta_rank) * C::kCtaM + warp * 32;
      // Element offsets of this lane's row in C and D (the batch entry selects the batch stride).
      // Reduce-scatter: row of this lane inside its slice, and the rows of the receive buffers it reads / writes.
      const int32_t rs_row_in_slice = RS ? (ti.tm_walk % p.rs_tiles_per_slice) * C::kTileM + int32_t(cta_rank) * C::kCtaM + warp * 32 : 0;
      const int64_t c_row_off = RS ? int64_t(p.rs_parity_rows + (rs_stage - 1) * p.rs_slice_rows + rs_row_in_slice + lane) * p.N
                                   : int64_t(ti.map_l) * p.batch_stride_c + int64_t(warp_map_row0 + lane) * ldc;
      const int64_t d_row_off = int64_t(ti.map_l) * p.batch_stride_d + int64_t(warp_map_row0 + lane) * ldd;
      const uint32_t lane_addr = tmem_base + (uint32_t(warp * 32) << 16) + acc_col;
      const bool reverse = (BN == 256) && ((it & 1) == 0);
      const uint32_t empty_bar = tempty0 + acc_bar * 8;
      // This warp's 32 rows lie inside the group: the output goes through shared memory and TMA stores.  (A TMA
      // store clips at the end of the matrix, not at the end of a group: the warp that holds a group's last rows
      // stores them row by row.)
      const int out_kind = p.out_kind;
      const bool quantised = OUTX ? out_is_quantised(out_kind) : out_kind != kOutBf16;
      const bool col_major = OUTX && quantised && p.out_col_major != 0;
      // (Pointer-array form: every group has a map of its own, which clips at the group's last row.)
      const bool tma_out = (PTR ? cta_row0 + warp * 32 < ti.row_end : cta_row0 + warp * 32 + 32 <= ti.row_end) && !col_major;
      // Staging sub-buffers a warp cycles through (4 KB per warp): bf16 uses all of it per 64 columns, e4m3 half,
      // e2m1 a quarter; a sub-buffer is rewritten once all but the newest n_bufs - 1 stores have read theirs.
      const int n_bufs = !quantised ? 1 : out_kind == kOutMxfp8 ? 2 : 4;

#pragma unroll 1
      for (int pi = 0; pi < n_pairs; ++pi) {
        const int pr = reverse ? (n_pairs - 1 - pi) : pi;
        uint32_t v[2][32];
        ptx::tmem_ld_32x32b_x32(lane_addr + pr * 64, v[0]);
        ptx::tmem_ld_32x32b_x32(lane_addr + pr * 64 + 32, v[1]);
        ptx::tmem_ld_wait();
        if (warp == 0 && pi == 0) BSG_DBG(2, 22);
        if (pi == C::kReleasePair) {
          ptx::tc_fence_before();
          __syncwarp();
          // Relaxed arrival: the reads of the accumulator columns have completed (wait::ld above), and an
          // arrival with release semantics was measured to stall this lane until its TMA stores of the previous
          // tile had drained (about 1 700 cycles per tile, during which the MMA warp waits for the accumulator).
          if (lane == 0) {
            if constexpr (CG == 2) ptx::mbar_arrive_remote_relaxed(ptx::mapa(empty_bar, 0));
            else ptx::mbar_arrive_relaxed(empty_bar);
          }
          if (warp == 0) BSG_DBG(2, 21);
        }
        uint8_t* sub_buf = stage_buf + (n_store % n_bufs) * (4096 / n_bufs);
        if (tma_out) ++n_store;      // counts the stores actually issued: the wait below is in units of those
        if (tma_out) {
          // The store that last used this sub-buffer must have finished reading it before it is overwritten.
          if (lane == 0) {
            if (n_bufs == 1) ptx::bulk_wait_group_read<0>();
            else if (n_bufs == 2) ptx::bulk_wait_group_read<1>();
            else ptx::bulk_wait_group_read<3>();
          }
          __syncwarp();
        }
        uint32_t sf_pair = 0;       // quantised outputs: the scale-factor codes of this lane's row for these 64 columns
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int32_t col0 = tile_col0 + pr * 64 + h * 32;
          const int32_t cols_valid = prob_N - col0;
          if (cols_valid <= 0 || (!row_ok && !tma_out)) continue;

          float x[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __fmul_rn(alpha, __uint_as_float(v[h][j]));
          if (p.bias_mode == 1) {
            const float* b = p.bias + int64_t(ti.g) * p.bias_group_stride + col0;
            if (cols_valid >= 32) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 bv = __ldg(reinterpret_cast<const float4*>(b) + q);
                x[q * 4 + 0] = __fadd_rn(x[q * 4 + 0], bv.x); x[q * 4 + 1] = __fadd_rn(x[q * 4 + 1], bv.y);
                x[q * 4 + 2] = __fadd_rn(x[q * 4 + 2], bv.z); x[q * 4 + 3] = __fadd_rn(x[q * 4 + 3], bv.w);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (j < cols_valid) x[j] = __fadd_rn(x[j], __ldg(b + j));
              }
            }
          } else if (p.bias_mode == 2 && row_ok) {
            const float bv = __ldg(p.bias + lrow);
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = __fadd_rn(x[j], bv);
          }
          if (use_c && row_ok) {
            const __nv_bfloat16* crow = (RS ? p.rs_recv : Cg) + c_row_off + col0;
            const float beta_c = RS ? 1.0f : beta;
            if (cols_valid >= 32) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                // Reduce-scatter: the addend was written by another GPU during this kernel: no read-only cache path.
                const uint4 cv = RS ? ld_global_v4(reinterpret_cast<const uint4*>(crow) + q) : __ldg(reinterpret_cast<const uint4*>(crow) + q);
                const uint32_t w[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float c_lo = __uint_as_float(w[e] << 16);
                  const float c_hi = __uint_as_float(w[e] & 0xFFFF0000u);
                  x[q * 8 + e * 2 + 0] = __fadd_rn(__fmul_rn(beta_c, c_lo), x[q * 8 + e * 2 + 0]);
                  x[q * 8 + e * 2 + 1] = __fadd_rn(__fmul_rn(beta_c, c_hi), x[q * 8 + e * 2 + 1]);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (j < cols_valid) x[j] = __fadd_rn(__fmul_rn(beta_c, __uint_as_float(uint32_t(*reinterpret_cast<const volatile uint16_t*>(crow + j)) << 16)), x[j]);
              }
            }
          }

          if (p.activation != kActIdentity) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = apply_activation(x[j], p.activation);
          }

          if (col_major) {
            // Column-major quantised output (the reference's Sm100BlockScaleFactorColStore,
            // include/cutlass/epilogue/fusion/sm100_visitor_store_tma_warpspecialized.hpp:352): blocks run along M.
            // The warp's 32 x 32 values are transposed through its staging buffer (128-byte rows, 16-byte chunks
            // XOR-swizzled by the row index), after which lane n owns column col0 + n with its 32 rows, and the
            // row-major arithmetic applies unchanged.  M is a multiple of 32, so a warp's rows are all valid or none.
            float* tb = reinterpret_cast<float*>(stage_buf);
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j) tb[j * 32 + ((((lane >> 2) ^ (j & 7)) << 2) | (lane & 3))] = x[j];
            __syncwarp();
            float y[32];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 v4 = *reinterpret_cast<const float4*>(tb + lane * 32 + ((i ^ (lane & 7)) << 2));
              y[4 * i + 0] = v4.x; y[4 * i + 1] = v4.y; y[4 * i + 2] = v4.z; y[4 * i + 3] = v4.w;
            }
            __syncwarp();
            const int32_t col = col0 + lane;
            const int32_t m0 = lrow - lane;                                  // first row of the warp's slab (multiple of 32)
            const int32_t m_k_atoms = ((p.rows_per_group + sfd_vec - 1) / sfd_vec + 3) / 4;
            if (col < prob_N && grow - lane < ti.row_end) {
              uint8_t* sf_base = SFDg + int64_t(col / 128) * (512ll * m_k_atoms) + 16 * (col & 31) + 4 * ((col & 127) >> 5);
              if (out_kind == kOutNvfp4) {
                uint32_t packed[4];
                uint32_t codes = 0;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                  float amax = 0.f;
#pragma unroll
                  for (int j = 0; j < 16; ++j) amax = ptx::fmax_nan(amax, fabsf(y[b * 16 + j]));
                  const uint32_t q = ptx::cvt_ue4m3(__fmul_rn(amax, st_scaled));
                  float sc = __fmul_rn(st, __fdiv_rn(1.0f, ptx::cvt_e4m3_to_f32(q)));
                  sc = ptx::fmin_nan(sc, FLT_MAX);
                  codes |= q << (8 * b);
#pragma unroll
                  for (int e = 0; e < 2; ++e) {
                    float z[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) z[j] = __fmul_rn(y[b * 16 + e * 8 + j], sc);
                    packed[b * 2 + e] = ptx::cvt_e2m1x8(z);
                  }
                }
                *reinterpret_cast<uint4*>(Dg + (int64_t(col) * ldd + m0) / 2) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                const int32_t mb = m0 >> 4;                                  // even: the two blocks share a 16-bit word
                *reinterpret_cast<uint16_t*>(sf_base + (mb >> 2) * 512 + (mb & 3)) = uint16_t(codes);
              } else {
                float amax = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) amax = ptx::fmax_nan(amax, fabsf(y[j]));
                const uint32_t q = ptx::cvt_ue8m0_rp(__fmul_rn(amax, st_scaled));
                float sc = __fmul_rn(st, __fdiv_rn(1.0f, ptx::ue8m0_to_f32(q)));
                sc = ptx::fmin_nan(sc, FLT_MAX);
                uint32_t w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  w[e] = ptx::cvt_e4m3x4(__fmul_rn(y[e * 4 + 0], sc), __fmul_rn(y[e * 4 + 1], sc), __fmul_rn(y[e * 4 + 2], sc), __fmul_rn(y[e * 4 + 3], sc));
                uint4* dcol = reinterpret_cast<uint4*>(Dg + int64_t(col) * ldd + m0);
                dcol[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dcol[1] = make_uint4(w[4], w[5], w[6], w[7]);
                const int32_t mb = m0 >> 5;
                sf_base[(mb >> 2) * 512 + (mb & 3)] = uint8_t(q);
              }
            }
          } else if (OUTX && out_kind == kOutF32) {
            // fp32 output: 32 columns are 128 bytes, so each half of the pair fills the staging tile (128-byte swizzle:
            // 16-byte chunk c of row r lives at chunk c ^ (r & 7)) and leaves with a store of its own.
            if (tma_out) {
              if (h == 1) {
                if (lane == 0) ptx::bulk_wait_group_read<0>();
                __syncwarp();
              }
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(stage_buf + lane * 128 + ((q ^ (lane & 7)) * 16)) = make_float4(x[q * 4], x[q * 4 + 1], x[q * 4 + 2], x[q * 4 + 3]);
              if (h == 0) {
                ptx::fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                  ptx::tma_store_3d(mapD, ptx::smem_u32(stage_buf), col0, warp_map_row0, ti.map_l);
                  ptx::bulk_commit_group();
                }
              }
            } else {
              float* drow = reinterpret_cast<float*>(Dg) + d_row_off + col0;
              if (cols_valid >= 32) {
#pragma unroll
                for (int q = 0; q < 8; ++q) reinterpret_cast<float4*>(drow)[q] = make_float4(x[q * 4], x[q * 4 + 1], x[q * 4 + 2], x[q * 4 + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (j < cols_valid) drow[j] = x[j];
                }
              }
            }
          } else if (out_kind == kOutBf16) {
            if (tma_out) {
              // 128-byte-swizzled staging tile: 16-byte chunk c of row r lives at chunk (c ^ (r & 7)).
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack_bf16x2(x[q * 8 + 0], x[q * 8 + 1]);
                o.y = pack_bf16x2(x[q * 8 + 2], x[q * 8 + 3]);
                o.z = pack_bf16x2(x[q * 8 + 4], x[q * 8 + 5]);
                o.w = pack_bf16x2(x[q * 8 + 6], x[q * 8 + 7]);
                const int chunk = (h * 4 + q) ^ (lane & 7);
                *reinterpret_cast<uint4*>(stage_buf + lane * 128 + chunk * 16) = o;
              }
            } else {
              __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(Dg) + d_row_off + col0;
              if (cols_valid >= 32) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 o;
                  o.x = pack_bf16x2(x[q * 8 + 0], x[q * 8 + 1]);
                  o.y = pack_bf16x2(x[q * 8 + 2], x[q * 8 + 3]);
                  o.z = pack_bf16x2(x[q * 8 + 4], x[q * 8 + 5]);
                  o.w = pack_bf16x2(x[q * 8 + 6], x[q * 8 + 7]);
                  reinterpret_cast<uint4*>(drow)[q] = o;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (j < cols_valid) drow[j] = __float2bfloat16_rn(x[j]);
                }
              }
            }
          } else if (OUTX && out_kind == kOutF16) {
            // as bf16, with the other 16-bit conversion
            if (tma_out) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 o = make_uint4(pack_f16x2(x[q * 8 + 0], x[q * 8 + 1]), pack_f16x2(x[q * 8 + 2], x[q * 8 + 3]),
                                           pack_f16x2(x[q * 8 + 4], x[q * 8 + 5]), pack_f16x2(x[q * 8 + 6], x[q * 8 + 7]));
                *reinterpret_cast<uint4*>(stage_buf + lane * 128 + (((h * 4 + q) ^ (lane & 7)) * 16)) = o;
              }
            } else {
              __half* drow = reinterpret_cast<__half*>(Dg) + d_row_off + col0;
              if (cols_valid >= 32) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  reinterpret_cast<uint4*>(drow)[q] = make_uint4(pack_f16x2(x[q * 8 + 0], x[q * 8 + 1]), pack_f16x2(x[q * 8 + 2], x[q * 8 + 3]),
                                                                 pack_f16x2(x[q * 8 + 4], x[q * 8 + 5]), pack_f16x2(x[q * 8 + 6], x[q * 8 + 7]));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (j < cols_valid) drow[j] = __float2half_rn(x[j]);
                }
              }
            }
          } else if (OUTX && (out_kind == kOutE4m3 || out_kind == kOutE5m2)) {
            // 8-bit floating-point output without scale factors: round to nearest even, saturating
            uint32_t w[8];
            if (out_kind == kOutE4m3) {
#pragma unroll
              for (int e = 0; e < 8; ++e) w[e] = ptx::cvt_e4m3x4(x[e * 4 + 0], x[e * 4 + 1], x[e * 4 + 2], x[e * 4 + 3]);
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) w[e] = ptx::cvt_e5m2x4(x[e * 4 + 0], x[e * 4 + 1], x[e * 4 + 2], x[e * 4 + 3]);
            }
            if (tma_out) {
              // 64-byte rows, 64-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ ((r >> 1) & 3).
              const int sw = (lane >> 1) & 3;
              *reinterpret_cast<uint4*>(sub_buf + lane * 64 + (((h * 2 + 0) ^ sw) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
              *reinterpret_cast<uint4*>(sub_buf + lane * 64 + (((h * 2 + 1) ^ sw) * 16)) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
              uint8_t* drow = Dg + d_row_off + col0;
              if (cols_valid >= 16) reinterpret_cast<uint4*>(drow)[0] = make_uint4(w[0], w[1], w[2], w[3]);
              if (cols_valid >= 32) reinterpret_cast<uint4*>(drow)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          } else if (out_kind == kOutMxfp8) {
            // MXFP8 re-quantisation: one ue8m0 scale factor (round-up conversion) for the 32 columns of
            // this row held here, e4m3 values; same routine of the reference host GEMM as below.
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) amax = ptx::fmax_nan(amax, fabsf(x[j]));     // NaN propagates, as in the reference
            const float pv = __fmul_rn(amax, st_scaled);
            const uint32_t q = ptx::cvt_ue8m0_rp(pv);
            float sc = __fmul_rn(st, __fdiv_rn(1.0f, ptx::ue8m0_to_f32(q)));
            sc = ptx::fmin_nan(sc, FLT_MAX);
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              w[e] = ptx::cvt_e4m3x4(__fmul_rn(x[e * 4 + 0], sc), __fmul_rn(x[e * 4 + 1], sc), __fmul_rn(x[e * 4 + 2], sc),
                                     __fmul_rn(x[e * 4 + 3], sc));
            if (cols_valid >= 32) sf_pair |= q << (8 * h);
            if (tma_out) {
              // 64-byte rows, 64-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ ((r >> 1) & 3).
              const int sw = (lane >> 1) & 3;
              *reinterpret_cast<uint4*>(sub_buf + lane * 64 + (((h * 2 + 0) ^ sw) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
              *reinterpret_cast<uint4*>(sub_buf + lane * 64 + (((h * 2 + 1) ^ sw) * 16)) = make_uint4(w[4], w[5], w[6], w[7]);
            } else if (cols_valid >= 32) {
              uint8_t* drow = Dg + d_row_off + col0;
              reinterpret_cast<uint4*>(drow)[0] = make_uint4(w[0], w[1], w[2], w[3]);
              reinterpret_cast<uint4*>(drow)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          } else {
            // NVFP4 re-quantisation, one scale factor per 16 columns of this row; same
            // operation order as compute_1d_scaling_factor_and_quantized_output of the
            // reference host GEMM (tools/util/include/cutlass/util/reference/host/gett.hpp:364-481).
            uint32_t packed[4];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              float amax = 0.f;
#pragma unroll
              for (int j = 0; j < 16; ++j) amax = ptx::fmax_nan(amax, fabsf(x[b * 16 + j]));   // NaN propagates, as in the reference
              const float pv = __fmul_rn(amax, st_scaled);
              const uint32_t q = ptx::cvt_ue4m3(pv);
              const float qf = ptx::cvt_e4m3_to_f32(q);
              float sc = __fmul_rn(st, __fdiv_rn(1.0f, qf));
              sc = ptx::fmin_nan(sc, FLT_MAX);
              if (cols_valid >= 16 * (b + 1)) sf_pair |= q << (16 * h + 8 * b);
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                float y[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) y[j] = __fmul_rn(x[b * 16 + e * 8 + j], sc);
                packed[b * 2 + e] = ptx::cvt_e2m1x8(y);
              }
            }
            if (tma_out) {
              // 32-byte rows, no swizzle: a warp's 32 rows fill 1 KB back to back.
              *reinterpret_cast<uint4*>(sub_buf + lane * 32 + h * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
              uint8_t* drow = Dg + (d_row_off + col0) / 2;
              if (cols_valid >= 32) *reinterpret_cast<uint4*>(drow) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              else if (cols_valid >= 16) *reinterpret_cast<uint2*>(drow) = make_uint2(packed[0], packed[1]);
            }
          }
        }
        if (quantised && !col_major && row_ok && tile_col0 + pr * 64 < prob_N) {
          // Scale factors of this row for the 64 columns: consecutive bytes of one 512-byte atom of the interleaved
          // layout (4 per row for 16-wide blocks, 2 for 32-wide ones).
          const int32_t pair_col0 = tile_col0 + pr * 64;
          const int32_t cols_left = prob_N - pair_col0;
          const int32_t nb = pair_col0 / sfd_vec;
          uint8_t* sfp = SFDg + (int64_t(ti.group_atom0) + lrow / 128) * (512ll * sfd_k_atoms) + (nb >> 2) * 512 +
                         16 * (lrow & 31) + 4 * ((lrow & 127) >> 5) + (nb & 3);
          if (out_kind == kOutNvfp4) {
            if (cols_left >= 64) *reinterpret_cast<uint32_t*>(sfp) = sf_pair;
            else {
#pragma unroll
              for (int b = 0; b < 4; ++b) if (cols_left >= 16 * (b + 1)) sfp[b] = uint8_t(sf_pair >> (8 * b));
            }
          } else {
            if (cols_left >= 64) *reinterpret_cast<uint16_t*>(sfp) = uint16_t(sf_pair);
            else if (cols_left >= 32) sfp[0] = uint8_t(sf_pair);
          }
        }
        if (tma_out) {
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            // Column coordinate in bytes / elements of the D map: bf16 elements, e4m3 bytes, two e2m1 per byte.
            const int32_t col = tile_col0 + pr * 64;
            if (RS && rs_to_peer)
              ptx::tma_store_3d(&tmDpeer, ptx::smem_u32(sub_buf), col, p.rs_parity_rows + rs_stage * p.rs_slice_rows + rs_row_in_slice, 0);
            else if (RS && p.rs_allreduce) {
              if (!dead) {
                for (int q = 0; q < p.rs_world; ++q)
                  ptx::tma_store_3d(p.rs_out_maps + q, ptx::smem_u32(sub_buf), col, p.rs_rank * p.rs_slice_rows + rs_row_in_slice, p.rs_out_half);
              }
            } else if (RS)
              ptx::tma_store_3d(&tmD, ptx::smem_u32(sub_buf), col, rs_row_in_slice, 0);
            else
              ptx::tma_store_3d(mapD, ptx::smem_u32(sub_buf), out_kind == kOutNvfp4 ? col / 2 : (OUTX && out_kind == kOutF32) ? col + 32 : col, warp_map_row0, ti.map_l);
            ptx::bulk_commit_group();
          }
        }
      }
      if constexpr (RS) {
        // Announce this warp's part of the tile to rank - 1: its stores must be complete (not only read from shared
        // memory) and ordered before the counter, in the form the memory model asks for.
        if (rs_to_peer && lane == 0 && !dead) {
          ptx::bulk_wait_group<0>();
          asm volatile("fence.proxy.async;" ::: "memory");
          asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(rs_flag_out), "r"(1u) : "memory");
        }
        // All-reduce: this warp's part of a finished tile is in every rank's output once its stores are complete.
        if (!rs_to_peer && p.rs_allreduce && p.rs_world > 1 && lane == 0 && !dead) {
          ptx::bulk_wait_group<0>();
          asm volatile("fence.proxy.async;" ::: "memory");
          for (int q = 0; q < p.rs_world; ++q) {
            if (q != p.rs_rank)
              asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.rs_peer_sync[q] + kRsSyncArrived), "r"(1u) : "memory");
          }
        }
      }
      ++it;
    }
    if (lane == 0) ptx::bulk_wait_group<0>();
    if constexpr (RS) {
      // All-reduce: the kernel ends only when the other ranks' slices have arrived, so that whatever follows on the
      // stream finds the whole result (one thread of the grid waits; bounded).
      if (p.rs_allreduce && p.rs_world > 1 && blockIdx.x == 0 && warp == 0 && lane == 0 && !dead) {
        if (!wait_flag_ge(p.rs_sync + kRsSyncArrived, p.rs_done_target, ctl)) atomicOr(p.status, kStTimeoutPeer);
      }
    }
    if (dead) atomicOr(p.status, kStTimeoutTmemFull);
  }

  // ------------------------------------------------------------------ teardown
  if (ctl->abort) {
    // Give copies and MMAs that may still be in flight time to land before the CTA's
    // shared and tensor memory are handed back.
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000ll) __nanosleep(1000);
  }
  __syncwarp();
  ptx::tc_fence_before();
  if constexpr (CG == 2) { ptx::cluster_arrive(); ptx::cluster_wait(); } else { __syncthreads(); }
  if (warp == 4) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<CG>(tmem_base, 512);
  }
#ifdef BSG_PROFILE
  if (dbg_on) {
    uint32_t* dbg_g = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(p.status) + 1024);
    for (int i = threadIdx.x; i < 512 + 1024 + 256; i += blockDim.x) dbg_g[i] = dbg_s[i];
  }
#endif
}

}  // namespace bsg
