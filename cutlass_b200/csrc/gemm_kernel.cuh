// Persistent warp-specialised block-scaled GEMM for sm_100a.
//
//   D = alpha * (A . SFA)(B . SFB)^T + beta * C          (bf16 out), or
//   (D, SFD) = nvfp4_quantise(alpha * ... + beta * C)     (e2m1 + ue4m3 out)
//
// One kernel serves the dense, batched, grouped (ragged M) and flag-gated
// (tensor-parallel) forms: every output tile belongs to a "group" that owns a
// contiguous run of rows of A and D, one B matrix and one pair of scale-factor
// layouts.
//
// Roles (192 threads): warps 0-3 epilogue (TMEM lane quadrant = warp id),
// warp 4 UMMA issue + TMEM allocation, warp 5 TMA producer.  With CG == 2 two
// CTAs of a cluster form one 256-row MMA (cta_group::2): both load their half
// of A and B, the even CTA issues the MMA, both run their own epilogue.
//
// This takes the place of the reference kernel
// include/cutlass/gemm/kernel/sm100_gemm_tma_warpspecialized.hpp together with the
// mainloop include/cutlass/gemm/collective/sm100_blockscaled_mma_warpspecialized.hpp
// (load :879, mma :949) and the linear-combination / block-scale-factor epilogue
// (include/cutlass/epilogue/fusion/sm100_visitor_store_tma_warpspecialized.hpp:226-275).
// Every wait is bounded: on a timeout the kernel records a status bit, drains and returns.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cfloat>
#include <cstdint>

#include "ptx.cuh"

namespace bsg {

constexpr int kMaxGroups = 256;
constexpr int kKindNvfp4 = 0;
constexpr int kKindMxfp8 = 1;
constexpr int kOutBf16 = 0;
constexpr int kOutNvfp4 = 1;

// Bits of the device status word.
constexpr uint32_t kStTimeoutFull = 1u;       // MMA warp: operands never arrived
constexpr uint32_t kStTimeoutEmpty = 2u;      // producer: stage never released
constexpr uint32_t kStTimeoutTmemFull = 4u;   // epilogue: accumulator never completed
constexpr uint32_t kStTimeoutTmemEmpty = 8u;  // MMA warp: accumulator never drained
constexpr uint32_t kStTimeoutFlag = 16u;      // producer: row-ready flag never set
constexpr uint32_t kStBadOffsets = 32u;       // grouped: offsets not monotone / out of range

struct GemmParams {
  int32_t num_groups;         // 1 for a dense GEMM
  int32_t rows_per_group;     // dense / batched: M of every group (offsets == nullptr)
  int32_t total_rows;         // rows of A and D over all groups
  int32_t N, K;
  const int32_t* offsets;     // grouped: cumulative END row of each group (device)
  int32_t b_rows_per_group;   // row distance between the B matrices of two groups (0: shared B)
  int32_t sfb_atoms_per_group;
  int32_t tiles_n;
  int32_t raster_band;
  int32_t out_kind;
  const __nv_bfloat16* C;
  void* D;
  uint8_t* SFD;
  int64_t ldc, ldd;           // elements
  float alpha, beta;
  const float* alpha_ptr;
  const float* beta_ptr;
  const float* norm_ptr;
  uint32_t* status;
  // Optional gating of A rows by flags (tensor-parallel all-gather): rows
  // [i*rows_per_flag, (i+1)*rows_per_flag) may be read once ready_flags[i] >= flag_target.
  const uint32_t* ready_flags;
  int32_t rows_per_flag;
  uint32_t flag_target;
  int32_t tile_m_rotate;      // dense only: start the M sweep at this tile row
};

template <int KIND, int CG, int BN>
struct Cfg {
  static_assert(KIND == kKindNvfp4 || KIND == kKindMxfp8, "kind");
  static_assert(CG == 1 || CG == 2, "cta group");
  static_assert(BN == 128 || BN == 256, "tile n");
  static constexpr int kCtaM = 128;                       // accumulator rows per CTA (= TMEM lanes)
  static constexpr int kTileM = kCtaM * CG;               // rows per MMA tile
  static constexpr int kRowBytes = 128;                   // bytes of K per row per k-tile (one 128B swizzle atom)
  static constexpr int kTileK = KIND == kKindNvfp4 ? 256 : 128;   // elements of K per k-tile
  static constexpr int kMmaK = KIND == kKindNvfp4 ? 64 : 32;      // elements of K per instruction (32 bytes)
  static constexpr int kSfVec = KIND == kKindNvfp4 ? 16 : 32;
  static constexpr int kKAtoms = KIND == kKindNvfp4 ? 4 : 1;      // 512-byte SF atoms along K per k-tile
  static constexpr int kBRowsCta = BN / CG;               // rows of B each CTA loads
  static constexpr int kABytes = kCtaM * kRowBytes;
  static constexpr int kBBytes = kBRowsCta * kRowBytes;
  static constexpr int kSfaBytes = kKAtoms * 512;
  static constexpr int kSfbBytes = (BN / 128) * kKAtoms * 512;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kCtlBytes = 8192;
  static constexpr int kSmemLimit = 232448;               // 227 KB
  static constexpr int kStagesRaw = (kSmemLimit - kCtlBytes - 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + kCtlBytes + 1024;
  // TMEM columns: two accumulators (overlapping by 48 columns when BN == 256), then SFA, then SFB.
  static constexpr int kAccStride = BN == 256 ? 208 : 128;
  static constexpr int kAccBars = BN == 256 ? 1 : 2;
  static constexpr int kSfaCol = 464;
  static constexpr int kSfbCol = 480;
  static constexpr int kChunks = BN / 32;
  static constexpr int kReleaseChunk = BN == 256 ? 1 : kChunks - 1;   // chunk after whose load the accumulator is released
};

struct alignas(8) Ctl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  volatile uint32_t abort;
  int32_t total_tiles;
  int32_t pad;
  int32_t tile_start[kMaxGroups + 1];
  int32_t row0[kMaxGroups];
  int32_t rows[kMaxGroups];
  int32_t atom0[kMaxGroups];
};
static_assert(sizeof(Ctl) <= 8192, "control block too large");

struct TileInfo {
  int32_t g, tm, tn;
  int32_t row0;       // first row of the tile in A / D
  int32_t row_end;    // end row of the group
  int32_t group_row0; // first row of the group
  int32_t sf_atom;    // SFA / SFD row-atom index of the tile's first row
};

__device__ __forceinline__ TileInfo decode_tile(const Ctl* ctl, const GemmParams& p, int32_t t, int32_t tile_m) {
  int lo = 0, hi = p.num_groups;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (ctl->tile_start[mid] <= t) lo = mid; else hi = mid;
  }
  TileInfo ti;
  ti.g = lo;
  const int32_t local = t - ctl->tile_start[lo];
  const int32_t rows = ctl->rows[lo];
  const int32_t tiles_m = (rows + tile_m - 1) / tile_m;
  const int32_t band = p.raster_band;
  const int32_t per_band = band * p.tiles_n;
  const int32_t b = local / per_band;
  const int32_t rem = local - b * per_band;
  const int32_t bh = min(band, tiles_m - b * band);
  int32_t tm = b * band + rem % bh;
  ti.tn = rem / bh;
  if (p.tile_m_rotate != 0) tm = (tm + p.tile_m_rotate) % tiles_m;
  ti.tm = tm;
  ti.group_row0 = ctl->row0[lo];
  ti.row0 = ti.group_row0 + tm * tile_m;
  ti.row_end = ti.group_row0 + rows;
  ti.sf_atom = ctl->atom0[lo] + tm * (tile_m / 128);
  return ti;
}

// Bounded mbarrier wait.  Returns false (and raises the CTA abort flag and a status bit) on timeout.
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, Ctl* ctl, uint32_t* status, uint32_t code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      const uint64_t limit = ctl->abort ? 20000ull : 2000000000ull;   // 20 us once aborting, else 2 s
      if (ptx::globaltimer_ns() - t0 > limit) break;
    }
  }
  ctl->abort = 1;
  atomicOr(status, code);
  return false;
}

__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart (SBO), LBO unused (1), descriptor version 1.
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t smem_addr) {
  // Un-swizzled K-major 32 rows x 16 bytes: 8-row groups 128 bytes apart.
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (8ull << 32) | (1ull << 46);
}

template <int KIND, int CG, int BN>
__device__ __forceinline__ uint32_t make_idesc() {
  constexpr uint32_t fmt = KIND == kKindNvfp4 ? 1u : 0u;       // E2M1 (mxf4) / E4M3 (mxf8f6f4)
  constexpr uint32_t sf_fmt = KIND == kKindNvfp4 ? 0u : 1u;    // UE4M3 / UE8M0
  constexpr uint32_t m = 128u * CG;
  return (fmt << 7) | (fmt << 10) | ((uint32_t(BN) >> 3) << 17) | (sf_fmt << 23) | ((m >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int KIND, int CG, int BN>
__global__ void __launch_bounds__(192, 1)
bsg_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                const GemmParams p) {
  using C = Cfg<KIND, CG, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + C::kStages * C::kABytes;
  uint8_t* sSFA = sB + C::kStages * C::kBBytes;
  uint8_t* sSFB = sSFA + C::kStages * C::kSfaBytes;
  Ctl* ctl = reinterpret_cast<Ctl*>(sSFB + C::kStages * C::kSfbBytes);

  const int warp = threadIdx.x >> 5;
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
    ptx::mbar_init(ptx::smem_u32(&ctl->drain), 1);
    ctl->abort = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async();
  }
  if (warp == 5 && lane == 0) {
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
    ptx::prefetch_tmap(&tmSFA);
    ptx::prefetch_tmap(&tmSFB);
  }
  // Group table: end rows first (parallel), then a serial prefix by one thread.
  for (int g = threadIdx.x; g < p.num_groups; g += blockDim.x) {
    ctl->rows[g] = p.offsets ? p.offsets[g] : (g + 1) * p.rows_per_group;   // holds END rows for now
  }
  __syncthreads();
  if (threadIdx.x == 32) {
    int32_t prev_end = 0, tiles = 0, atoms = 0;
    bool bad = false;
    for (int g = 0; g < p.num_groups; ++g) {
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

  const uint32_t tmem_base = ctl->tmem_base;
  const int32_t total_tiles = ctl->total_tiles;
  const int32_t k_tiles = (p.K + C::kTileK - 1) / C::kTileK;

  if (warp == 5) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int32_t t = cluster_idx; t < total_tiles && ok; t += num_clusters) {
        const TileInfo ti = decode_tile(ctl, p, t, C::kTileM);
        const int32_t a_row = ti.row0 + int32_t(cta_rank) * C::kCtaM;
        const int32_t b_row = ti.g * p.b_rows_per_group + ti.tn * BN + int32_t(cta_rank) * C::kBRowsCta;
        // The second CTA of a pair may lie wholly past the group's last row: keep its
        // scale-factor fetch inside the group's own atoms (its rows are never stored).
        const int32_t group_atoms = (ti.row_end - ti.group_row0 + 127) >> 7;
        const int32_t sfa_atom = min(ti.sf_atom + int32_t(cta_rank), ctl->atom0[ti.g] + max(group_atoms, 1) - 1);
        const int32_t sfb_atom = ti.g * p.sfb_atoms_per_group + ti.tn * (BN / 128);
        if (p.ready_flags != nullptr) {
          const uint32_t* flag = p.ready_flags + ti.row0 / p.rows_per_flag;
          const uint64_t t0 = ptx::globaltimer_ns();
          while (ptx::ld_acquire_sys_u32(flag) < p.flag_target) {
            if (ptx::globaltimer_ns() - t0 > 2000000000ull || ctl->abort) {
              ctl->abort = 1;
              atomicOr(p.status, kStTimeoutFlag);
              ok = false;
              break;
            }
            __nanosleep(64);
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int32_t kt = 0; kt < k_tiles; ++kt) {
          if (!bounded_wait(ptx::smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.status, kStTimeoutEmpty)) {
            ok = false;
            break;
          }
          const uint32_t full_local = ptx::smem_u32(&ctl->full[stage]);
          if (is_leader) ptx::mbar_arrive_expect_tx(full_local, uint32_t(C::kStageBytes) * CG);
          const uint32_t bar = CG == 2 ? ptx::mapa(full_local, 0) : full_local;
          ptx::tma_load_2d<CG>(ptx::smem_u32(sA + stage * C::kABytes), &tmA, bar, kt * C::kRowBytes, a_row);
          ptx::tma_load_2d<CG>(ptx::smem_u32(sB + stage * C::kBBytes), &tmB, bar, kt * C::kRowBytes, b_row);
          ptx::tma_load_3d<CG>(ptx::smem_u32(sSFA + stage * C::kSfaBytes), &tmSFA, bar, 0, kt * C::kKAtoms, sfa_atom);
          ptx::tma_load_3d<CG>(ptx::smem_u32(sSFB + stage * C::kSfbBytes), &tmSFB, bar, 0, kt * C::kKAtoms, sfb_atom);
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
      // Tail: every stage must have been released, so that no commit-arrive is still
      // in flight towards this CTA's shared memory when it exits.
      for (int s = 0; s < C::kStages && ok; ++s) {
        ok = bounded_wait(ptx::smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.status, kStTimeoutEmpty);
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 4) {
    // ---------------------------------------------------------------- UMMA issue
    if (is_leader && lane == 0) {
      const uint32_t idesc = make_idesc<KIND, CG, BN>();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int32_t it = 0;
      for (int32_t t = cluster_idx; t < total_tiles && ok; t += num_clusters, ++it) {
        const int acc_bar = it % C::kAccBars;
        const uint32_t acc_phase = uint32_t(it / C::kAccBars) & 1u;
        const uint32_t d_tmem = tmem_base + uint32_t(it & 1) * C::kAccStride;
        if (!bounded_wait(ptx::smem_u32(&ctl->tmem_empty[acc_bar]), acc_phase ^ 1u, ctl, p.status, kStTimeoutTmemEmpty)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        for (int32_t kt = 0; kt < k_tiles; ++kt) {
          if (!bounded_wait(ptx::smem_u32(&ctl->full[stage]), phase, ctl, p.status, kStTimeoutFull)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sfa_s = ptx::smem_u32(sSFA + stage * C::kSfaBytes);
          const uint32_t sfb_s = ptx::smem_u32(sSFB + stage * C::kSfbBytes);
#pragma unroll
          for (int ka = 0; ka < C::kKAtoms; ++ka) {
            ptx::utccp_32x128b_warpx4<CG>(tmem_base + C::kSfaCol + 4 * ka, make_desc_sf(sfa_s + ka * 512));
          }
#pragma unroll
          for (int ra = 0; ra < BN / 128; ++ra) {
#pragma unroll
            for (int ka = 0; ka < C::kKAtoms; ++ka) {
              ptx::utccp_32x128b_warpx4<CG>(tmem_base + C::kSfbCol + (BN / 32) * ka + 4 * ra,
                                            make_desc_sf(sfb_s + (ra * C::kKAtoms + ka) * 512));
            }
          }
          const uint64_t a_desc = make_desc_sw128(ptx::smem_u32(sA + stage * C::kABytes));
          const uint64_t b_desc = make_desc_sw128(ptx::smem_u32(sB + stage * C::kBBytes));
          const int32_t k_left = p.K - kt * C::kTileK;
          const int n_mma = k_left >= C::kTileK ? 4 : (k_left + C::kMmaK - 1) / C::kMmaK;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            if (kb < n_mma) {
              uint32_t sfa_t, sfb_t, id = idesc;
              if constexpr (KIND == kKindNvfp4) {
                sfa_t = tmem_base + C::kSfaCol + 4 * kb;
                sfb_t = tmem_base + C::kSfbCol + (BN / 32) * kb;
              } else {
                sfa_t = tmem_base + C::kSfaCol;
                sfb_t = tmem_base + C::kSfbCol;
                id |= (uint32_t(kb) << 4) | (uint32_t(kb) << 29);   // scale-factor byte of this K block
              }
              ptx::umma_block_scaled<KIND, CG>(d_tmem, a_desc + 2 * kb, b_desc + 2 * kb, id, sfa_t, sfb_t,
                                               (kt > 0 || kb > 0) ? 1u : 0u);
            }
          }
          ptx::umma_commit<CG>(ptx::smem_u32(&ctl->empty[stage]));
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::umma_commit<CG>(ptx::smem_u32(&ctl->tmem_full[acc_bar]));
      }
      if (!ok) {
        // Drain: nothing issued by this thread may still be running at teardown.
        ptx::umma_commit<CG>(ptx::smem_u32(&ctl->drain));
        bounded_wait(ptx::smem_u32(&ctl->drain), 0, ctl, p.status, 0);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (warps 0-3)
    const float alpha = p.alpha_ptr ? *p.alpha_ptr : p.alpha;
    const float beta = p.beta_ptr ? *p.beta_ptr : p.beta;
    const bool use_c = (p.C != nullptr) && (beta != 0.0f);
    float st = 0.f, st_scaled = 0.f;
    if (p.out_kind == kOutNvfp4) {
      st = *p.norm_ptr;
      st_scaled = __fmul_rn(st, __fdiv_rn(1.0f, 6.0f));
    }
    const int32_t sfd_k_atoms = ((p.N + 15) / 16 + 3) / 4;
    const uint32_t tmem_empty0 = ptx::smem_u32(&ctl->tmem_empty[0]);
    bool ok = true;
    int32_t it = 0;
    for (int32_t t = cluster_idx; t < total_tiles && ok; t += num_clusters, ++it) {
      const TileInfo ti = decode_tile(ctl, p, t, C::kTileM);
      const int acc_bar = it % C::kAccBars;
      const uint32_t acc_phase = uint32_t(it / C::kAccBars) & 1u;
      const uint32_t acc_col = uint32_t(it & 1) * C::kAccStride;
      ok = bounded_wait(ptx::smem_u32(&ctl->tmem_full[acc_bar]), acc_phase, ctl, p.status, kStTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();

      const int32_t grow = ti.row0 + int32_t(cta_rank) * C::kCtaM + warp * 32 + lane;
      const bool row_ok = grow < ti.row_end;
      const int32_t lrow = grow - ti.group_row0;
      const uint32_t lane_addr = tmem_base + (uint32_t(warp * 32) << 16) + acc_col;
      const bool reverse = (BN == 256) && ((it & 1) == 0);
      const uint32_t empty_bar = tmem_empty0 + acc_bar * 8;

#pragma unroll 1
      for (int ci = 0; ci < C::kChunks; ++ci) {
        const int c = reverse ? (C::kChunks - 1 - ci) : ci;
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(lane_addr + c * 32, v);
        ptx::tmem_ld_wait();
        if (ci == C::kReleaseChunk) {
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CG == 2) ptx::mbar_arrive_remote(ptx::mapa(empty_bar, 0));
            else ptx::mbar_arrive(empty_bar);
          }
        }
        const int32_t col0 = ti.tn * BN + c * 32;
        const int32_t cols_valid = p.N - col0;
        if (!row_ok || cols_valid <= 0) continue;

        float x[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = __fmul_rn(alpha, __uint_as_float(v[j]));
        if (use_c) {
          const __nv_bfloat16* crow = p.C + int64_t(grow) * p.ldc + col0;
          if (cols_valid >= 32) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 cv = __ldg(reinterpret_cast<const uint4*>(crow) + q);
              const uint32_t w[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                const float c_lo = __uint_as_float(w[h] << 16);
                const float c_hi = __uint_as_float(w[h] & 0xFFFF0000u);
                x[q * 8 + h * 2 + 0] = __fadd_rn(__fmul_rn(beta, c_lo), x[q * 8 + h * 2 + 0]);
                x[q * 8 + h * 2 + 1] = __fadd_rn(__fmul_rn(beta, c_hi), x[q * 8 + h * 2 + 1]);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < cols_valid) x[j] = __fadd_rn(__fmul_rn(beta, __bfloat162float(crow[j])), x[j]);
            }
          }
        }

        if (p.out_kind == kOutBf16) {
          __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + int64_t(grow) * p.ldd + col0;
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
        } else {
          // NVFP4 re-quantisation, one scale factor per 16 columns of this row; same
          // operation order as compute_1d_scaling_factor_and_quantized_output of the
          // reference host GEMM (tools/util/include/cutlass/util/reference/host/gett.hpp:364-481).
          uint8_t* drow = reinterpret_cast<uint8_t*>(p.D) + (int64_t(grow) * p.ldd + col0) / 2;
          uint32_t packed[4];
          uint32_t sf_codes = 0;
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(x[b * 16 + j]));
            const float pv = __fmul_rn(amax, st_scaled);
            const uint32_t q = ptx::cvt_ue4m3(pv);
            const float qf = ptx::cvt_e4m3_to_f32(q);
            float sc = __fmul_rn(st, __fdiv_rn(1.0f, qf));
            sc = fminf(sc, FLT_MAX);
            sf_codes |= q << (8 * b);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              float y[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) y[j] = __fmul_rn(x[b * 16 + h * 8 + j], sc);
              packed[b * 2 + h] = ptx::cvt_e2m1x8(y);
            }
          }
          const int32_t nb = col0 >> 4;
          uint8_t* sfp = p.SFD + (int64_t(ctl->atom0[ti.g]) + lrow / 128) * (512ll * sfd_k_atoms) + (nb >> 2) * 512 +
                         16 * (lrow & 31) + 4 * ((lrow & 127) >> 5) + (nb & 3);
          if (cols_valid >= 32) {
            *reinterpret_cast<uint4*>(drow) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            *reinterpret_cast<uint16_t*>(sfp) = uint16_t(sf_codes);
          } else if (cols_valid >= 16) {
            *reinterpret_cast<uint2*>(drow) = make_uint2(packed[0], packed[1]);
            *sfp = uint8_t(sf_codes);
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (ctl->abort) {
    // Give copies and MMAs that may still be in flight time to land before the CTA's
    // shared and tensor memory are handed back.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  __syncwarp();
  ptx::tc_fence_before();
  if constexpr (CG == 2) { ptx::cluster_arrive(); ptx::cluster_wait(); } else { __syncthreads(); }
  if (warp == 4) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<CG>(tmem_base, 512);
  }
}

}  // namespace bsg
