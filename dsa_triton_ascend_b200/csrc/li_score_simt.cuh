// Portable (CUDA-core) lightning-indexer score kernel: any head count, head dim and layout.
// Computes what _lightning_indexer_score_kernel does (lightning_indexer_triton.py:154-284)
// for the visible prefix of every row; positions outside the prefix are never written
// because the top-k stage derives the same prefix length and never reads them.
#pragma once

#include "dsa_common.cuh"

namespace dsa {

struct LiDev {
  SeqDesc seq;
  const void* query;
  const void* key;
  const void* weights;
  int32_t* out_indices;
  void* out_values;
  int32_t dtype_w;
  int32_t n1, n2, d;
  int32_t rows;  // number of query rows (batch * s1 or T1)
  int32_t sparse_count, rank_mode, return_value;
};

constexpr int kSimtKeys = 128;   // keys per block (one per thread)
constexpr int kSimtHeads = 16;   // heads accumulated per pass
constexpr int kSimtDims = 64;    // head-dim slice staged in shared memory
constexpr int kSimtKStride = kSimtDims + 4;

// grid = (rows * n2, ceil(s2 / 128)); block = 128 threads, thread t owns key tile*128 + t.
template <typename T>
__global__ void __launch_bounds__(kSimtKeys) li_score_simt_kernel(LiDev p, float* __restrict__ scores,
                                                                   int64_t ld) {
  __shared__ __align__(16) float ks[kSimtKeys * kSimtKStride];
  __shared__ __align__(16) float qs[kSimtHeads * kSimtDims];

  const int32_t rown = blockIdx.x;
  const int32_t row = rown / p.n2;
  const int32_t n2 = rown - row * p.n2;
  const RowInfo ri = row_info(p.seq, row);
  const int32_t tile0 = blockIdx.y * kSimtKeys;
  if (tile0 >= ri.visible) return;

  const int32_t group = p.n1 / p.n2;
  const int32_t tid = threadIdx.x;
  const int32_t pos = tile0 + tid;
  const T* kq = (const T*)p.key;
  const T* qq = (const T*)p.query + (int64_t)row * p.n1 * p.d;
  int64_t krow = (pos < ri.visible) ? key_row(p.seq, ri, pos) : -1;
  const T* kptr = krow >= 0 ? kq + (krow * p.n2 + n2) * (int64_t)p.d : nullptr;

  float total = 0.f;
  for (int g0 = 0; g0 < group; g0 += kSimtHeads) {
    float acc[kSimtHeads];
#pragma unroll
    for (int g = 0; g < kSimtHeads; ++g) acc[g] = 0.f;
    for (int d0 = 0; d0 < p.d; d0 += kSimtDims) {
      __syncthreads();
      // stage this thread's key slice and the head chunk's query slice as fp32 (zero padded)
      for (int i = 0; i < kSimtDims; ++i) {
        int dd = d0 + i;
        ks[tid * kSimtKStride + i] = (kptr != nullptr && dd < p.d) ? to_f32<T>(kptr[dd]) : 0.f;
      }
      for (int i = tid; i < kSimtHeads * kSimtDims; i += kSimtKeys) {
        int g = i / kSimtDims, dd = d0 + (i - g * kSimtDims);
        int head = n2 * group + g0 + g;
        qs[i] = (g0 + g < group && dd < p.d) ? to_f32<T>(qq[(int64_t)head * p.d + dd]) : 0.f;
      }
      __syncthreads();
      const float4* k4 = reinterpret_cast<const float4*>(&ks[tid * kSimtKStride]);
#pragma unroll 4
      for (int i = 0; i < kSimtDims / 4; ++i) {
        float4 kv = k4[i];
#pragma unroll
        for (int g = 0; g < kSimtHeads; ++g) {
          float4 qv = reinterpret_cast<const float4*>(&qs[g * kSimtDims])[i];
          acc[g] = fmaf(kv.x, qv.x, acc[g]);
          acc[g] = fmaf(kv.y, qv.y, acc[g]);
          acc[g] = fmaf(kv.z, qv.z, acc[g]);
          acc[g] = fmaf(kv.w, qv.w, acc[g]);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < kSimtHeads; ++g) {
      if (g0 + g < group) {
        float wv = load_weight(p.weights, p.dtype_w, (int64_t)row * p.n1 + n2 * group + g0 + g);
        // separate multiply and add, as the golden's `scores += relu * w` rounds twice
        total = __fadd_rn(total, __fmul_rn(fmaxf(acc[g], 0.f), wv));
      }
    }
  }
  if (pos < ri.visible) scores[(int64_t)rown * ld + pos] = total + 0.f;
}

}  // namespace dsa
