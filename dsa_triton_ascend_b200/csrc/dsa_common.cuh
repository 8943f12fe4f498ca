// Shared device-side helpers: sequence/row bookkeeping for the three layouts (BSND, TND,
// paged cache) and io-dtype conversion.  The reference normalises TND and paged inputs to
// dense BSND with host copy loops (lightning_indexer_triton.py:294-340,
// sparse_flash_attention_triton.py:975-1033); here every kernel derives the same addresses
// from the row number instead.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dsa_b200.h"

#include <atomic>

namespace dsa {

// Kernels this library has launched in this process (read by dsa_kernel_launch_count()).
inline std::atomic<unsigned long long>& launch_counter() {
  static std::atomic<unsigned long long> n{0};
  return n;
}
inline void count_launch(unsigned k = 1) { launch_counter().fetch_add(k, std::memory_order_relaxed); }

// Sequence description shared by both operators (device copy of the ABI struct fields).
struct SeqDesc {
  const int32_t* seq_q;
  const int32_t* seq_k;
  const int32_t* block_table;
  int32_t layout_q, layout_k;
  int32_t seq_q_cum, seq_k_cum;
  int32_t batch, s1, s2;
  int32_t block_size, max_blocks;
  int32_t sparse_mode;
  int64_t key_rows;   // physical key rows behind the key pointer (0: unknown, no check)
};

// Everything a kernel needs to know about one query row.
struct RowInfo {
  int32_t b;          // sequence (batch entry) of the row
  int32_t pos;        // position of the row inside its sequence
  int32_t act_q;      // valid query length of the sequence
  int32_t act_k;      // valid key length of the sequence
  int32_t threshold;  // keys < threshold are causally visible (before the act_k clip)
  int32_t visible;    // min(threshold, act_k, s2) clipped at 0; 0 for inactive rows
  int64_t key_base;   // first key row of the sequence (BSND / TND); unused for paged keys
};

__device__ __forceinline__ RowInfo row_info(const SeqDesc& s, int32_t row) {
  RowInfo r;
  int32_t start_q = 0;
  if (s.layout_q == DSA_LAYOUT_TND) {
    // seq_q holds cumulative ends; find the sequence that owns this token.
    int32_t lo = 0, hi = s.batch - 1;
    while (lo < hi) {
      int32_t mid = (lo + hi) >> 1;
      if (row < s.seq_q[mid]) hi = mid; else lo = mid + 1;
    }
    r.b = lo;
    start_q = lo > 0 ? s.seq_q[lo - 1] : 0;
    r.pos = row - start_q;
    r.act_q = s.seq_q[lo] - start_q;
  } else {
    r.b = row / s.s1;
    r.pos = row - r.b * s.s1;
    if (s.seq_q == nullptr) r.act_q = s.s1;
    else if (s.seq_q_cum) r.act_q = s.seq_q[r.b] - (r.b > 0 ? s.seq_q[r.b - 1] : 0);
    else r.act_q = s.seq_q[r.b];
  }
  int32_t start_k = 0;
  if (s.seq_k == nullptr) {
    r.act_k = s.s2;
  } else if (s.seq_k_cum) {
    start_k = r.b > 0 ? s.seq_k[r.b - 1] : 0;
    r.act_k = s.seq_k[r.b] - start_k;
  } else {
    r.act_k = s.seq_k[r.b];
  }
  r.key_base = (s.layout_k == DSA_LAYOUT_TND) ? (int64_t)start_k : (int64_t)r.b * s.s2;
  r.threshold = (s.sparse_mode == 3) ? (r.act_k - r.act_q + r.pos + 1) : r.act_k;
  int32_t vis = min(min(r.threshold, r.act_k), s.s2);
  r.visible = (r.pos < r.act_q && vis > 0) ? vis : 0;
  return r;
}

// Physical key row of logical position `p` of sequence r.b; -1 (the callers read a zero row) when a
// paged block is absent or when the row would lie outside the key tensor: a stale block-table entry
// or cumulative lengths that overrun the tensor must not become an out-of-bounds read.
__device__ __forceinline__ int64_t key_row(const SeqDesc& s, const RowInfo& r, int32_t p) {
  int64_t row;
  if (s.layout_k == DSA_LAYOUT_PA_BSND) {
    int32_t blk_i = p / s.block_size;
    if (blk_i >= s.max_blocks) return -1;
    int32_t blk = s.block_table[(int64_t)r.b * s.max_blocks + blk_i];
    if (blk < 0) return -1;
    row = (int64_t)blk * s.block_size + (p - blk_i * s.block_size);
  } else {
    row = r.key_base + p;
  }
  if (s.key_rows > 0 && row >= s.key_rows) return -1;
  return row;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Round-trip through the io dtype (round to nearest even).
template <typename T> __device__ __forceinline__ float round_io(float v) { return to_f32<T>(from_f32<T>(v)); }

__device__ __forceinline__ float load_weight(const void* w, int32_t dtype_w, int64_t i) {
  if (dtype_w == DSA_DTYPE_FP32) return ((const float*)w)[i];
  if (dtype_w == DSA_DTYPE_FP16) return __half2float(((const __half*)w)[i]);
  return __bfloat162float(((const __nv_bfloat16*)w)[i]);
}

}  // namespace dsa
