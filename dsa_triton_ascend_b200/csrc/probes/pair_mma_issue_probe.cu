// Probe behind the attention kernel's issuer layout: how fast can pair MMAs (cta_group::2, M = 128)
// be issued by one thread, and do several issuing warps overlap?  Streams of N = 64 / 80 / 96 / 128
// (K-major B) and N = 256 (MN-major B) MMAs from one, two or three warps, alone and mixed in the
// proportions of an attention tile (36 score MMAs : 8 value MMAs per 64 keys).
// Build and run (one B200):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o pair_mma_issue_probe pair_mma_issue_probe.cu && ./pair_mma_issue_probe
#include <cstdio>
#include <cstdint>
#include <cuda_bf16.h>
#include "../ptx_sm100.cuh"
using namespace dsa;
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t t, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(t), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma2_ss(uint32_t d, uint64_t ad, uint64_t bd, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d), "l"(ad), "l"(bd), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void commit2(uint64_t* bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(ptx::smem_u32(bar)), "h"(mask) : "memory");
}
constexpr int kSm = 8192 + 16384 + 16384;   // A 8 KB | B kmajor 16 KB | B mn-major 16 KB
// One issuer stream: `tiles` tiles of `nmma` MMAs each (4 k-steps cycling), unrolled by 4.
template <int kN, bool kMn>
__device__ __forceinline__ void stream(uint32_t d, uint32_t a0, uint32_t b0, int nmma_total) {
  const uint32_t id = ptx::idesc_f16(1, 128, kN, 0, kMn ? 1 : 0);
  uint64_t ad[4], bd[4];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    ad[ks] = ptx::desc_kmajor_sw128(a0 + ks * 32);
    bd[ks] = kMn ? ptx::desc_mnmajor_sw128(b0 + ks * 2048, 8192, 1024) : ptx::desc_kmajor_sw128(b0 + ks * 32);
  }
  for (int n = 0; n < nmma_total; n += 4) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) mma2_ss(d, ad[ks], bd[ks], id, 1u);
  }
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) probe2(long long* tim) {
  extern __shared__ __align__(1024) unsigned char sm[];
  __shared__ uint64_t bar[4];
  __shared__ uint32_t tmem_slot;
  __shared__ int abortf;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool report = (blockIdx.x >> 1) == 0;
  if (threadIdx.x == 0) { for (int i = 0; i < 4; ++i) ptx::mbar_init(&bar[i], 1); abortf = 0; ptx::mbar_fence_init(); }
  if (warp == 0) { tmem_alloc2(&tmem_slot, 512); tmem_relinquish2(); }
  for (int i = threadIdx.x; i < kSm / 4; i += 128) reinterpret_cast<uint32_t*>(sm)[i] = 0x3c003c00u;
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_slot;
  ptx::cluster_arrive(); ptx::cluster_wait();
  const uint32_t a0 = ptx::smem_u32(sm), bk = ptx::smem_u32(sm + 8192), bm = ptx::smem_u32(sm + 8192 + 16384);
  bool ok = true;
  uint32_t phase = 0;
  const int R = 1024;
  // cfg 0..4: single issuer (warp 0): N=64, 80, 96, 128 kmajor, N=256 mn
  // cfg 5: two issuers N=64 (warps 0,1) ; cfg 6: two issuers N=128 ; cfg 7: warps 0,1 N=64 + warp 2 N=256mn (R/4 MMAs... ratio 36:8 -> R and R*8/36)
  // cfg 8: warp 0 N=128 + warp 2 N=256mn (ratio 36:16) ; cfg 9: warp 0 N=64 + warp 2 N=256 mn (36:8) ; cfg 10: warps 0,1 N=80 + warp2 N=256mn (36:10)
  for (int cfg = 0; cfg < 11 && ok; ++cfg) {
    __syncthreads();
    long long t0 = clock64();
    if (rank == 0 && lane == 0) {
      bool mine = false;
      if (cfg < 5) {
        if (warp == 0) {
          mine = true;
          if (cfg == 0) stream<64, false>(tmem, a0, bk, R);
          else if (cfg == 1) stream<80, false>(tmem, a0, bk, R);
          else if (cfg == 2) stream<96, false>(tmem, a0, bk, R);
          else if (cfg == 3) stream<128, false>(tmem, a0, bk, R);
          else stream<256, true>(tmem + 256, a0, bm, R);
        }
      } else if (cfg == 5) {
        if (warp < 2) { mine = true; stream<64, false>(tmem + warp * 64, a0, bk, R); }
      } else if (cfg == 6) {
        if (warp < 2) { mine = true; stream<128, false>(tmem + warp * 64, a0, bk, R); }
      } else if (cfg == 7) {
        if (warp < 2) { mine = true; stream<64, false>(tmem + warp * 64, a0, bk, R / 2); }
        if (warp == 2) { mine = true; stream<256, true>(tmem + 256, a0, bm, R * 8 / 36 / 4 * 4); }
      } else if (cfg == 8) {
        if (warp == 0) { mine = true; stream<128, false>(tmem, a0, bk, R); }
        if (warp == 2) { mine = true; stream<256, true>(tmem + 256, a0, bm, R * 16 / 36 / 4 * 4); }
      } else if (cfg == 9) {
        if (warp == 0) { mine = true; stream<64, false>(tmem, a0, bk, R); }
        if (warp == 2) { mine = true; stream<256, true>(tmem + 256, a0, bm, R * 8 / 36 / 4 * 4); }
      } else if (cfg == 10) {
        if (warp < 2) { mine = true; stream<80, false>(tmem + warp * 64, a0, bk, R / 2); }
        if (warp == 2) { mine = true; stream<256, true>(tmem + 256, a0, bm, R * 10 / 36 / 4 * 4); }
      }
      const long long ti = clock64();
      if (mine) commit2(&bar[warp], 3);
      else ptx::mbar_arrive(&bar[warp]);
      if (report) tim[32 + cfg * 4 + warp] = ti - t0;
    } else if (lane == 0) {
      if (rank != 0) {
        // the peer's barriers get the multicast arrival only from issuing warps; arrive for the others
        bool mine = (cfg < 5) ? warp == 0 : (cfg == 5 || cfg == 6) ? warp < 2 : (cfg == 7 || cfg == 10) ? warp < 3 : (warp == 0 || warp == 2);
        if (!mine) ptx::mbar_arrive(&bar[warp]);
      }
    }
    __syncwarp();
    ok = __all_sync(0xffffffffu, ptx::mbar_wait(&bar[warp], phase & 1, &abortf));
    ++phase;
    __syncthreads();
    if (report && rank == 0 && threadIdx.x == 0) tim[cfg] = clock64() - t0;
    ok = __syncthreads_and(ok);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive(); ptx::cluster_wait();
  ptx::tc_fence_after();
  if (warp == 0) tmem_dealloc2(tmem, 512);
}
int main() {
  long long* tim;
  cudaMalloc(&tim, 128 * 8);
  cudaMemset(tim, 0, 128 * 8);
  cudaFuncSetAttribute(probe2, cudaFuncAttributeMaxDynamicSharedMemorySize, kSm);
  probe2<<<148, 128, kSm>>>(tim);
  cudaError_t e = cudaDeviceSynchronize();
  printf("probe2: %s\n", cudaGetErrorString(e));
  if (e != cudaSuccess) return 1;
  long long h[128];
  cudaMemcpy(h, tim, sizeof(h), cudaMemcpyDeviceToHost);
  const char* names[11] = {"1 issuer N=64 x1024", "1 issuer N=80 x1024", "1 issuer N=96 x1024", "1 issuer N=128 x1024", "1 issuer N=256mn x1024",
                           "2 issuers N=64 x1024 each", "2 issuers N=128 x1024 each", "2 x N=64 x512 + N=256mn x224", "N=128 x1024 + N=256mn x452",
                           "N=64 x1024 + N=256mn x224", "2 x N=80 x512 + N=256mn x284"};
  for (int i = 0; i < 11; ++i)
    printf("%-36s total %8lld cycles; issue times per warp: %lld %lld %lld\n", names[i], h[i], h[32 + i * 4], h[32 + i * 4 + 1], h[32 + i * 4 + 2]);
  return 0;
}
