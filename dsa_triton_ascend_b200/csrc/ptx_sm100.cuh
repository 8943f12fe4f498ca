// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the tensor-core kernels use:
// mbarrier, TMA tile / gather4 loads, tcgen05 (TMEM allocation, MMA, commit, load, fences).
// Every wait is bounded: it gives up after a fixed number of polls and reports failure so the
// kernel can record a status word and leave instead of hanging the GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dsa {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity), "r"(8000u)  // suspend-time hint in ns
      : "memory");
  return done != 0;
}
// Bounded wait.  `abort_flag` (shared memory) lets the other warps of a CTA leave quickly once
// one of them has given up.  Returns false on timeout / abort.
constexpr uint32_t kWaitPolls = 1u << 20;  // x (up to) 8 us per poll: gives up within seconds
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kWaitPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// ---- thread-block clusters / distributed shared memory -----------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Address of this CTA's shared-memory location `p` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t raddr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(raddr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void st_cluster_v4_b32(uint32_t raddr, uint4 v) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(raddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Asynchronous 16-byte store into another CTA of the cluster; when the bytes have landed they are
// counted as transaction bytes on an mbarrier of the destination CTA (no wait on the sender side).
__device__ __forceinline__ void st_async_v4(uint32_t raddr, uint4 v, uint32_t raddr_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(raddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"(raddr_bar)
               : "memory");
}
// Arrive on an mbarrier of another CTA of the cluster; orders this thread's earlier (remote) writes.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t raddr_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(raddr_bar) : "memory");
}
// Bulk copy of `bytes` (multiple of 16) from this CTA's shared memory into another CTA of the
// cluster; completion is counted as transaction bytes on an mbarrier of the destination CTA.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t raddr_dst, const void* src, uint32_t bytes,
                                                  uint32_t raddr_bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(raddr_dst), "r"(smem_u32(src)), "r"(bytes), "r"(raddr_bar)
      : "memory");
}
// Remote arrive that publishes nothing (it only says "I have finished reading"): relaxed, so it
// does not wait for this thread's outstanding writes.  `dep` ties the instruction to a value that
// depends on the loads it must not overtake.
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t raddr_bar, uint32_t dep) {
  asm volatile(
      "{\n\t.reg .b32 t;\n\tand.b32 t, %1, 0;\n\tadd.u32 t, t, %0;\n\t"
      "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [t];\n\t}\n"
      ::"r"(raddr_bar), "r"(dep)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity), "r"(2000u)  // suspend-time hint in ns
      : "memory");
  return done != 0;
}

// Bounded wait on a barrier that another CTA of the cluster arrives on (cluster-scope acquire).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag);

// ---- proxies / fences -------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// all state spaces (covers rows written into a peer CTA's shared memory)
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < (kWaitPolls << 2); ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// Warp-wide waits: every lane polls.  Letting one lane poll and handing the result to the others
// with a shuffle or a warp barrier looks cheaper and is not: measured on B200, the lanes parked at
// the shuffle resumed ~1400 cycles after the polling lane had seen the barrier flip (whichever of
// try_wait / test_wait / sleep it used), which made a gather producer's tile 2.6x and the whole
// attention kernel 1.7x slower.  Must be called by all 32 lanes.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}
__device__ __forceinline__ bool mbar_wait_cluster_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait_cluster(bar, parity, abort_flag));
}

// Same, for hand-overs that are expected within a few hundred cycles: test_wait never suspends the
// thread, so the hand-over is seen without a wake-up delay (at the price of issue slots).
template <bool kCluster>
__device__ __forceinline__ bool mbar_spin_warp_impl(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  bool ok = false;
  for (uint32_t i = 0; i < (kWaitPolls << 6); ++i) {
    uint32_t done;
    if (kCluster) {
      asm volatile(
          "{\n\t.reg .pred P;\n\t"
          "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
          "selp.b32 %0, 1, 0, P;\n\t}\n"
          : "=r"(done)
          : "r"(smem_u32(bar)), "r"(parity)
          : "memory");
    } else {
      asm volatile(
          "{\n\t.reg .pred P;\n\t"
          "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
          "selp.b32 %0, 1, 0, P;\n\t}\n"
          : "=r"(done)
          : "r"(smem_u32(bar)), "r"(parity)
          : "memory");
    }
    if (done) { ok = true; break; }
    if ((i & 1023u) == 1023u && *abort_flag) break;
  }
  if (!ok && !*abort_flag) *abort_flag = 1;
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ bool mbar_spin_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return mbar_spin_warp_impl<false>(bar, parity, abort_flag);
}
__device__ __forceinline__ bool mbar_spin_cluster_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return mbar_spin_warp_impl<true>(bar, parity, abort_flag);
}

// ---- TMA ----------------------------------------------------------------------------------------
// 32-byte store (address 32-byte aligned)
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2D tile load: coordinates (x = innermost element, y = row).  x * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// 3D tile load: coordinates (x = innermost element, y, z).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int32_t x, int32_t y,
                                            int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Four rows (y0..y3) of one column box starting at x, gathered into four consecutive smem rows.
__device__ __forceinline__ void tma_gather4_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int32_t x, int32_t y0,
                                               int32_t y1, int32_t y2, int32_t y3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y0), "r"(y1),
      "r"(y2), "r"(y3)
      : "memory");
}

// ---- tcgen05: tensor memory ---------------------------------------------------------------------
// One warp allocates `cols` (power of two, 32..512) columns; the base address lands in *dst_smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// ---- tcgen05: MMA -------------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 128 bytes, groups
// of 8 rows 1024 bytes apart.  `addr` must point into a 1024-byte aligned tile (it may be
// advanced by 32-byte steps inside the swizzle atom to walk the K dimension).
__device__ __forceinline__ uint64_t desc_kmajor_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);        // start address
  d |= (uint64_t)1 << 16;                         // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset: 8 rows * 128 B
  d |= (uint64_t)1 << 46;                         // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
  return d;
}
// MN-major operand, 128-byte swizzle: 64 contiguous MN elements (128 B) per K row, 8 K rows per
// 1024-byte atom; `lbo` = bytes between consecutive 64-element MN blocks, `sbo` = bytes between
// consecutive groups of 8 K rows.
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor for kind::f16 (bf16 or fp16 inputs, fp32 accumulate).
// fmt: 0 = fp16, 1 = bf16.  a_mn / b_mn: 1 when the operand is MN-major.
__host__ __device__ constexpr uint32_t idesc_f16(uint32_t fmt, uint32_t m, uint32_t n, uint32_t a_mn, uint32_t b_mn) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem].
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- tcgen05 on a CTA pair (cta_group::2) ----------------------------------------------------------
// A pair is the two CTAs of a 2-CTA cluster.  One warp of EACH CTA allocates / frees (the same
// columns in both CTAs); one thread of the even-ranked CTA issues an MMA that runs on both tensor
// cores: each CTA contributes its own A rows (M/2) and half of B's N extent, read from the SAME
// shared-memory offsets in both CTAs, and accumulates its own M/2 rows of D.  With M = 128 the
// accumulator of a CTA sits in lanes 0..63 (row r, columns of the first half of N) and lanes
// 64..127 (row r again, second half of N), N/2 columns each (measured on B200).
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the mbarrier at this shared-memory offset in BOTH CTAs of the pair once all MMAs issued
// so far by this thread have completed.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}

// ---- tcgen05: TMEM loads (32 lanes x 32-bit, N consecutive columns per thread) --------------------
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

}  // namespace ptx

// ---- host side: tensor maps -----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved through the runtime, so the library carries no link-time
// dependency on libcuda and still loads on a machine without a driver.
inline EncodeTiledFn tensor_map_encoder() {
  // initialised once, thread-safe (function-local static)
  static const EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(p);
    return nullptr;
  }();
  return fn;
}

// 2D row-major 16-bit tensor [rows, cols] with a row pitch of `pitch_bytes`; box = [box_rows, box_cols];
// 128-byte swizzle (box_cols * 2 bytes must be 128).  Returns false when the driver refuses.
inline bool make_tmap_2d_16bit(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                               uint32_t box_rows, uint32_t box_cols, bool bf16) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 3D 16-bit tensor [d2, d1, cols] (cols innermost, contiguous; d1 rows `pitch1` bytes apart, d2
// slabs `pitch2` bytes apart); box = [1, box_rows, box_cols]; 128-byte swizzle.  Rows of the box
// past d1 read as zeros.
inline bool make_tmap_3d_16bit(CUtensorMap* m, const void* base, uint64_t d2, uint64_t d1, uint64_t cols,
                               uint64_t pitch1, uint64_t pitch2, uint32_t box_rows, uint32_t box_cols, bool bf16) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return false;
  cuuint64_t dims[3] = {cols, d1, d2};
  cuuint64_t strides[2] = {pitch1, pitch2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Same tensor, box of ONE row x box_cols: the form tile::gather4 loads take (each load names four
// row coordinates and brings 4 x box_cols elements).
inline bool make_tmap_gather4_16bit(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols,
                                    uint64_t pitch_bytes, uint32_t box_cols, bool bf16) {
  return make_tmap_2d_16bit(m, base, rows, cols, pitch_bytes, 1, box_cols, bf16);
}

}  // namespace dsa
