// Warp-level tensor-core building blocks (mma.sync m16n8k16 with fp32 accumulation, ldmatrix) shared by
// the kernels that work on tiles of 16 heads x a few keys: the attention backward, the indexer-loss
// kernels and the any-shape attention forward.  Fragment layouts (lane = 4 g + c):
//   A (16 x 16, row-major): a0 = (row g, cols 2c..2c+1), a1 = (row g+8, same), a2 / a3 = cols + 8
//   B (16 x 8, k x n):      b0 = (k 2c..2c+1, n g), b1 = (k 2c+8.., n g)
//   C (16 x 8):             c0, c1 = (row g, cols 2c, 2c+1), c2, c3 = (row g+8, same)
#pragma once

#include "dsa_common.cuh"

namespace dsa {

template <typename T>
constexpr bool kIsBf16 = false;
template <>
constexpr bool kIsBf16<__nv_bfloat16> = true;

template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// B fragment (16 x 8, k x n) of a row-major [k][n] tile in shared memory: rows k0 .. k0+15 start at
// `row0` (16-byte aligned, `stride` elements apart), columns n0 .. n0+7.
template <typename T>
__device__ __forceinline__ void ldmatrix_b_trans(uint32_t& b0, uint32_t& b1, const T* row0, int stride) {
  const int lane = threadIdx.x & 31;
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row0 + (lane & 15) * stride);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// A fragment (16 x 16, row-major rows m0 .. m0+15, columns k0 .. k0+15) by 32-bit loads.
template <typename T>
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const T* base, int stride, int m0, int k0) {
  const int lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  a[0] = *reinterpret_cast<const uint32_t*>(&base[(m0 + g) * stride + k0 + 2 * c]);
  a[1] = *reinterpret_cast<const uint32_t*>(&base[(m0 + g + 8) * stride + k0 + 2 * c]);
  a[2] = *reinterpret_cast<const uint32_t*>(&base[(m0 + g) * stride + k0 + 8 + 2 * c]);
  a[3] = *reinterpret_cast<const uint32_t*>(&base[(m0 + g + 8) * stride + k0 + 8 + 2 * c]);
}

}  // namespace dsa
