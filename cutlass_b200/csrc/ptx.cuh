// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA, tcgen05 (TMEM alloc,
// UMMA, UTCCP, loads, commit), cluster helpers.  One instruction per wrapper;
// no policy lives here.
//
// The same instructions appear in the reference as CuTe "arch" structs
// (include/cute/arch/mma_sm100_umma.hpp, copy_sm100.hpp, copy_sm100_tma.hpp,
// tmem_allocator_sm100.hpp, include/cutlass/arch/barrier.h); here they are
// written straight from the PTX ISA.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace bsg {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}

__device__ __forceinline__ uint32_t num_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}

// Address of `local_smem_addr` as seen in CTA `cta_rank` of this cluster.
__device__ __forceinline__ uint32_t mapa(uint32_t local_smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta_rank));
  return r;
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Programmatic dependent launch (no-ops unless the launch carries the programmatic-serialisation attribute):
// wait until the kernels this one depends on have completed and their writes are visible; allow the kernels
// that depend on this one to be scheduled.  The reference wraps the same instructions in
// include/cutlass/arch/grid_dependency_control.h:87,97.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Cluster launch control (the hardware's work stealing between the clusters of one grid): ask to cancel the launch of
// a cluster that has not started yet; the 16-byte answer lands in this CTA's shared memory at `response` (16-byte
// aligned) and completes 16 bytes on the mbarrier.  The reference issues the same request from its tile scheduler
// (include/cutlass/gemm/kernel/sm100_tile_scheduler.hpp:400).  One thread per cluster asks.
__device__ __forceinline__ void clc_try_cancel(uint32_t response, uint32_t bar) {
  asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
               ::"r"(response), "r"(bar)
               : "memory");
}
// Decodes an answer: x of the first CTA of the cancelled cluster, or 0xFFFFFFFF when nothing was cancelled (no
// cluster is left to start; no further request may be made after that).
__device__ __forceinline__ uint32_t clc_query_first_ctaid_x(uint32_t response) {
  uint32_t x, ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b128 r;\n\t"
      "ld.shared.b128 r, [%2];\n\t"
      "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, r;\n\t"
      "selp.u32 %1, 1, 0, p;\n\t"
      "mov.u32 %0, 0;\n\t"
      "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %0, r;\n\t"
      "}"
      : "=r"(x), "=r"(ok)
      : "r"(response)
      : "memory");
  return ok ? x : 0xFFFFFFFFu;
}
// 32-bit store into the shared memory of another CTA of the cluster (address from mapa).
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on a barrier that lives in another CTA of the cluster (address from mapa).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// The same arrivals without release semantics, for hand-overs whose data does not live in memory.
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Spin on a barrier phase inside one asm statement, so that the compiler sees straight-line,
// warp-uniform code.  Gives up after `tries` polls; returns 1 when the phase completed.
__device__ __forceinline__ uint32_t mbar_spin(uint32_t bar, uint32_t parity, uint32_t tries) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .u32 n;\n\t"
      "mov.u32 n, %3;\n\t"
      "SPIN_LOOP:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra SPIN_DONE;\n\t"
      "sub.u32 n, n, 1;\n\t"
      "setp.ne.u32 q, n, 0;\n\t"
      "@q bra SPIN_LOOP;\n\t"
      "SPIN_DONE:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(tries)
      : "memory");
  return ok;
}

// Same, polling with the non-blocking test_wait.
__device__ __forceinline__ uint32_t mbar_spin_test(uint32_t bar, uint32_t parity, uint32_t tries) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .u32 n;\n\t"
      "mov.u32 n, %3;\n\t"
      "SPIN_LOOP:\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra SPIN_DONE;\n\t"
      "sub.u32 n, n, 1;\n\t"
      "setp.ne.u32 q, n, 0;\n\t"
      "@q bra SPIN_LOOP;\n\t"
      "SPIN_DONE:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(tries)
      : "memory");
  return ok;
}

// True in exactly one lane of a fully active warp.
__device__ __forceinline__ uint32_t elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(pred));
  return pred;
}

// ---------------------------------------------------------------- TMA loads
// CG == 1: the barrier is in this CTA.  CG == 2: `bar` may be the leader CTA's
// barrier (cluster address); both CTAs of the pair signal it.
template <int CG>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int32_t c0, int32_t c1) {
  if constexpr (CG == 2) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
  }
}
template <int CG>
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int32_t c0, int32_t c1,
                                            int32_t c2) {
  if constexpr (CG == 2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
  }
}
// TMA store of one shared-memory box to global memory (bulk async-group completion).
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int32_t c0, int32_t c1, int32_t c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// Untiled bulk copies (addresses and size multiples of 16 bytes): global -> shared with mbarrier
// completion, and shared -> global (bulk async-group completion).
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until the bulk stores of all but the newest `N` groups have finished READING shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Wait until all but the newest `N` groups have completed entirely.
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// A tensor map that lies in global memory and was written there through the generic proxy (a copy from the host):
// the thread that hands it to the TMA engine first makes that write visible to the tensor-map proxy.
__device__ __forceinline__ void fence_tensormap_acquire(const void* tmap) {
  asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---------------------------------------------------------------- tcgen05
template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  if constexpr (CG == 2)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CG == 2)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CG == 2)
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// UTCCP: one 512-byte scale-factor atom (32 rows x 16 bytes) from shared memory
// into 4 TMEM columns, replicated over the four 32-lane quadrants.
template <int CG>
__device__ __forceinline__ void utccp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  if constexpr (CG == 2)
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
  else
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Block-scaled UMMA.  KIND 0: e2m1 x e2m1, ue4m3 scale per 16 (K = 64 per instruction).  KIND 2: the same data
// with ue8m0 scale per 32.  KIND 1 and 3: kind::mxf8f6f4 (8-bit containers; formats from the instruction
// descriptor) with ue8m0 scale per 32 (K = 32).
#define BSG_UMMA_ASM(CTA_GROUP, KIND_AND_SCALE)                                                                     \
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                                   \
               "tcgen05.mma.cta_group::" CTA_GROUP ".kind::" KIND_AND_SCALE " [%0], %1, %2, %3, [%5], [%6], p;\n\t}" \
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)  \
               : "memory")
template <int KIND, int CG>
__device__ __forceinline__ void umma_block_scaled(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if constexpr (KIND == 0) {
    if constexpr (CG == 2) BSG_UMMA_ASM("2", "mxf4nvf4.block_scale.block16");
    else BSG_UMMA_ASM("1", "mxf4nvf4.block_scale.block16");
  } else if constexpr (KIND == 2) {
    if constexpr (CG == 2) BSG_UMMA_ASM("2", "mxf4.block_scale.block32");
    else BSG_UMMA_ASM("1", "mxf4.block_scale.block32");
  } else {
    if constexpr (CG == 2) BSG_UMMA_ASM("2", "mxf8f6f4.block_scale");
    else BSG_UMMA_ASM("1", "mxf8f6f4.block_scale");
  }
}
#undef BSG_UMMA_ASM

// Arrive on `bar` (same shared-memory offset in every CTA of `cta_mask`) once all
// tcgen05 operations issued so far by this thread have completed.
template <int CG>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  if constexpr (CG == 2) {
    uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(mask)
        : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  }
}

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- conversions
// Two fp32 -> two e2m1 (round to nearest even, saturating); `lo` lands in bits [3:0].
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&x)[8]) {
  uint32_t out;
  asm volatile(
      "{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t"
      "}"
      : "=r"(out)
      : "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7]));
  return out;
}
// fp32 (>= 0) -> ue4m3 code, round to nearest even, saturating at 448.
__device__ __forceinline__ uint32_t cvt_ue4m3(float x) {
  uint16_t out;
  asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(out) : "f"(0.0f), "f"(x));
  return out & 0xFFu;
}
// e4m3 code -> fp32 (exact).
__device__ __forceinline__ float cvt_e4m3_to_f32(uint32_t code) {
  uint16_t in = static_cast<uint16_t>(code & 0xFFu);
  uint32_t h2;
  asm volatile("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half2float(__low2half(h));
}

// fp32 (>= 0) -> ue8m0 code, rounding up (float8.h:1174 of the reference uses the same instruction).  Infinity
// gives the NaN code 0xFF, as the reference's host conversion does (the format has no infinity; the instruction
// alone would saturate to the largest finite value).
__device__ __forceinline__ uint32_t cvt_ue8m0_rp(float x) {
  uint16_t out;
  asm volatile("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(out) : "f"(0.0f), "f"(x));
  return __float_as_uint(x) == 0x7F800000u ? 0xFFu : (out & 0xFFu);
}
// Maximum / minimum that return NaN when an operand is NaN (fmaxf / fminf return the other operand).
__device__ __forceinline__ float fmax_nan(float a, float b) {
  float d;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ float fmin_nan(float a, float b) {
  float d;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ float ue8m0_to_f32(uint32_t code) {
  if (code == 0xFFu) return __uint_as_float(0x7FC00000u);
  return code == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(code << 23);   // 2^(code - 127)
}
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return uint32_t(lo) | (uint32_t(hi) << 16);
}

// Cache prefetches of the line that holds `p` (no register is written, nothing waits).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

__device__ __forceinline__ uint32_t cvt_e5m2x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm volatile("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm volatile("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return uint32_t(lo) | (uint32_t(hi) << 16);
}

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

}  // namespace ptx
}  // namespace bsg
