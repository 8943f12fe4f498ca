// Probe behind the attention kernel's design: tcgen05.mma.cta_group::2 (pair MMA) with M = 128,
// i.e. 64 accumulator rows per CTA.
//  (1) where D[m][n] lands in each CTA's tensor memory (identity B operand, two fill patterns),
//  (2) cycles per MMA for N = 64 / 128 / 256 (K-major B) and N = 256 (MN-major B), and for the
//      MMA mix of a 64-key and of a 128-key attention tile, issued by one thread.
// Build and run (one B200):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o pair_mma_probe pair_mma_probe.cu && ./pair_mma_probe
// Every wait is bounded; the program allocates 512 tensor-memory columns per CTA and frees them.
#include <cstdio>
#include <cstdint>
#include <cstdlib>
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

constexpr int kA = 0;            // A tile: 64 rows x 64 K (8 KB)
constexpr int kB = 8192;         // B tile: up to 128 rows x 64 K (16 KB), or MN-major 64 keys x 128 cols
constexpr int kSm = 8192 + 16384;

__device__ __forceinline__ void put(unsigned char* tile, int r, int k, float v) {
  const uint32_t off = (r / 8) * 1024 + (r % 8) * 128 + (((k / 8) ^ (r % 8)) * 16) + (k % 8) * 2;
  *reinterpret_cast<__nv_bfloat16*>(tile + off) = __float2bfloat16(v);
}

// out: [2 ctas][2 tests][128 lanes][64 cols] floats, then timings
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
pair_probe(float* out, long long* tim, uint32_t* misc) {
  extern __shared__ __align__(1024) unsigned char sm[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abortf;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool report = (blockIdx.x >> 1) == 0;
  if (threadIdx.x == 0) { ptx::mbar_init(&bar, 1); abortf = 0; ptx::mbar_fence_init(); }
  if (warp == 0) { tmem_alloc2(&tmem_slot, 512); tmem_relinquish2(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (report && threadIdx.x == 0) misc[rank] = tmem;
  ptx::cluster_arrive(); ptx::cluster_wait();
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
  uint32_t phase = 0;
  bool ok = true;

  for (int test = 0; test < 2 && ok; ++test) {
    // prefill D region (cols 0..63) with -1
    {
      uint32_t v[32];
      for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(-1.f);
      ptx::tmem_st_x32(lane_addr + 0, v);
      ptx::tmem_st_x32(lane_addr + 32, v);
      ptx::tmem_st_wait();
    }
    // A_c[r][k]: test 0 -> global row 64*rank + r ; test 1 -> k
    for (int i = threadIdx.x; i < 64 * 64; i += 128) {
      const int r = i / 64, k = i % 64;
      put(sm + kA, r, k, test == 0 ? (float)(64 * rank + r) : (float)k);
    }
    // B_c[nl][k] = (32*rank + nl == k), N = 64 total, 32 rows per CTA
    for (int i = threadIdx.x; i < 32 * 64; i += 128) {
      const int nl = i / 64, k = i % 64;
      put(sm + kB, nl, k, (32 * (int)rank + nl == k) ? 1.f : 0.f);
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_arrive(); ptx::cluster_wait();
    ptx::tc_fence_after();
    if (rank == 0 && threadIdx.x == 0) {
      const uint32_t idesc = ptx::idesc_f16(1, 128, 64, 0, 0);
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t ad = ptx::desc_kmajor_sw128(ptx::smem_u32(sm + kA) + ks * 32);
        const uint64_t bd = ptx::desc_kmajor_sw128(ptx::smem_u32(sm + kB) + ks * 32);
        mma2_ss(tmem + 0, ad, bd, idesc, ks > 0 ? 1u : 0u);
      }
      commit2(&bar, 3);
    }
    ok = __all_sync(0xffffffffu, ptx::mbar_wait(&bar, phase & 1, &abortf));
    ++phase;
    if (ok) {
      ptx::tc_fence_after();
      uint32_t v[64];
      ptx::tmem_ld_x32(lane_addr + 0, v);
      ptx::tmem_ld_x32(lane_addr + 32, v + 32);
      ptx::tmem_ld_wait();
      if (report)
        for (int c = 0; c < 64; ++c)
          out[(((size_t)rank * 2 + test) * 128 + threadIdx.x) * 64 + c] = __uint_as_float(v[c]);
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_arrive(); ptx::cluster_wait();
    ptx::tc_fence_after();
  }

  // ---- timing (operands: whatever is in smem; zero them to keep values finite)
  for (int i = threadIdx.x; i < kSm / 4; i += 128) reinterpret_cast<uint32_t*>(sm)[i] = 0x3c003c00u;  // small bf16 values
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive(); ptx::cluster_wait();
  ptx::tc_fence_after();
  const int R = 512;
  // configs: 0: N=64 K-major, 1: N=128 K-major, 2: N=256 K-major, 3: N=256 MN-major,
  //          4: tile64 = 36 x N64 + 8 x N256mn ; 5: tile128 = 36 x N128 + 16 x N256mn
  for (int cfg = 0; cfg < 6 && ok; ++cfg) {
    long long t0 = 0, t1 = 0;
    if (rank == 0 && threadIdx.x == 0) {
      const uint32_t a0 = ptx::smem_u32(sm + kA), b0 = ptx::smem_u32(sm + kB);
      const uint32_t i64 = ptx::idesc_f16(1, 128, 64, 0, 0), i128 = ptx::idesc_f16(1, 128, 128, 0, 0),
                     i256 = ptx::idesc_f16(1, 128, 256, 0, 0), i256mn = ptx::idesc_f16(1, 128, 256, 0, 1);
      t0 = clock64();
      if (cfg < 4) {
        const uint32_t id = cfg == 0 ? i64 : cfg == 1 ? i128 : cfg == 2 ? i256 : i256mn;
        for (int n = 0; n < R; ++n) {
          const int ks = n & 3;
          const uint64_t ad = ptx::desc_kmajor_sw128(a0 + ks * 32);
          const uint64_t bd = cfg == 3 ? ptx::desc_mnmajor_sw128(b0 + ks * 2048, 8192, 1024) : ptx::desc_kmajor_sw128(b0 + ks * 32);
          mma2_ss(tmem + (cfg == 3 ? 256 : 0), ad, bd, id, 1u);
        }
      } else {
        const int nt = 16;
        for (int t = 0; t < nt; ++t) {
          for (int n = 0; n < 36; ++n) {
            const int ks = n & 3;
            mma2_ss(tmem + (t & 1) * 64, ptx::desc_kmajor_sw128(a0 + ks * 32), ptx::desc_kmajor_sw128(b0 + ks * 32),
                    cfg == 4 ? i64 : i128, n > 0 ? 1u : 0u);
          }
          const int npv = cfg == 4 ? 8 : 16;
          for (int n = 0; n < npv; ++n) {
            const int ks = (n >> 1) & 3;
            mma2_ss(tmem + 256, ptx::desc_kmajor_sw128(a0 + ks * 32), ptx::desc_mnmajor_sw128(b0 + ks * 2048, 8192, 1024), i256mn, 1u);
          }
        }
      }
      const long long ti = clock64();
      commit2(&bar, 3);
      if (report) tim[16 + cfg] = ti - t0;   // issue time
    }
    ok = __all_sync(0xffffffffu, ptx::mbar_wait(&bar, phase & 1, &abortf));
    ++phase;
    if (rank == 0 && threadIdx.x == 0) {
      t1 = clock64();
      if (report) tim[cfg] = t1 - t0;
    }
    __syncthreads();
  }
  if (report && threadIdx.x == 0) misc[2 + rank] = ok ? 1u : 0u;

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive(); ptx::cluster_wait();
  ptx::tc_fence_after();
  if (warp == 0) tmem_dealloc2(tmem, 512);
}

int main() {
  float* out; long long* tim; uint32_t* misc;
  cudaMalloc(&out, 2 * 2 * 128 * 64 * 4);
  cudaMalloc(&tim, 64 * 8);
  cudaMalloc(&misc, 64);
  cudaMemset(out, 0, 2 * 2 * 128 * 64 * 4);
  cudaMemset(tim, 0, 64 * 8);
  cudaMemset(misc, 0xff, 64);
  cudaFuncSetAttribute(pair_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, kSm);
  pair_probe<<<148, 128, kSm>>>(out, tim, misc);
  cudaError_t e = cudaDeviceSynchronize();
  printf("pair_probe: %s\n", cudaGetErrorString(e));
  if (e != cudaSuccess) return 1;
  static float h[2 * 2 * 128 * 64];
  long long ht[64]; uint32_t hm[16];
  cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
  cudaMemcpy(ht, tim, sizeof(ht), cudaMemcpyDeviceToHost);
  cudaMemcpy(hm, misc, sizeof(hm), cudaMemcpyDeviceToHost);
  printf("tmem base: cta0 %08x cta1 %08x ok %u %u\n", hm[0], hm[1], hm[2], hm[3]);
  for (int c = 0; c < 2; ++c)
    for (int t = 0; t < 2; ++t) {
      printf("== cta %d test %d (%s): lanes x cols (every 8th lane: cols 0,1,15,16,31,32,33,47,63)\n", c, t, t == 0 ? "D=row m" : "D=col n");
      for (int l = 0; l < 128; l += 8) {
        const float* r = h + (((size_t)c * 2 + t) * 128 + l) * 64;
        printf(" lane %3d: %5.0f %5.0f %5.0f %5.0f %5.0f %5.0f %5.0f %5.0f %5.0f | lane+1: %5.0f %5.0f\n", l, r[0], r[1], r[15], r[16], r[31], r[32], r[33],
               r[47], r[63], r[64], r[64 + 32]);
      }
    }
  const char* names[6] = {"N=64 kmajor", "N=128 kmajor", "N=256 kmajor", "N=256 mnmajor", "tile64 (36xN64+8xN256) x16", "tile128 (36xN128+16xN256) x16"};
  for (int i = 0; i < 6; ++i) {
    const double div = i < 4 ? 512.0 : 16.0;
    printf("pair M=128 %-32s total %8lld cycles -> %8.1f per %s (issue %8.1f)\n", names[i], ht[i], ht[i] / div, i < 4 ? "MMA" : "tile", ht[16 + i] / div);
  }
  return 0;
}
