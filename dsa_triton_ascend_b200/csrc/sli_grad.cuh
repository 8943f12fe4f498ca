// Backward of the sparse lightning indexer under the KL loss against the attention distribution
// (sparse_lightning_indexer_grad_kl_loss_triton.py:25-327, golden sli_grad_kl_loss_numpy.py:16-156).
// Per query row with n used slots and idx = its sparse indices clipped to [0, S2):
//     p[k]  = mean_h exp((q[h].k[idx k] + qr[h].kr[idx k]) * scale - max[h]) / (sum[h] + 1e-8)
//     I[k]  = sum_g w[g] relu(qi[g].ki[idx k]);  sI = softmax_k(I);  dI = sI - p
//     loss += sum_k max(p,1e-8) (log max(p,1e-8) - log max(sI,1e-8))
//     dW[g] = sum_k dI[k] relu[g,k];   ds[g,k] = dI[k] w[g] [relu[g,k] > 0]
//     dQI[g] = sum_k ds[g,k] ki[idx k];   dKI[idx k] += sum_g ds[g,k] qi[g]
// The reference runs all stages in one program per row and keeps ReLU values, gathered index keys,
// p, I and dI in global scratch tensors between them (:385-400).  Here: (1) one block per (row, 16
// heads) of either side keeps its heads in shared memory, walks over the row's keys 64 at a time,
// scores them on the tensor cores (mma.sync m16n8k16, fp32 accumulation) and adds its share of p[k]
// or I[k] into fp32 buffers; (2) one block per row turns I and p into dI and the row's loss term;
// (3) one block per (row, 16 index heads) recomputes the index scores it needs instead of reading a
// [rows, G, topK] ReLU cache, accumulates dQI in tensor-core accumulators and dW in registers, and
// adds its dKI tiles into an fp32 accumulator with 16-byte reductions; (4) the accumulator is
// converted and the loss terms are summed in a fixed order.
//
// The same kernels serve the dense operator (dense_loss_backward_triton.py:130-341: every causally
// visible key 0..n-1 instead of selected ones, attention keys with n2 heads, the student distribution
// normalised with index statistics given from outside) and, stopped after the index scores, the
// dense softmax-LSE helper (:344-420).
#pragma once

#include "dsa_common.cuh"
#include "sfa_bwd_mma.cuh"

namespace dsa {

struct SliGradDev {
  const void* query;        // [rows, n1, d]
  const void* query_rope;   // [rows, n1, d_rope] or null (d_rope 0)
  const void* key;          // [batch * s2, d]
  const void* key_rope;     // [batch * s2, d_rope] or null
  const void* query_index;  // [rows, g, d_idx]
  const void* key_index;    // [batch * s2, d_idx]
  const void* weights;      // [rows, g], dtype_w
  const int32_t* sparse_indices;   // [rows, topk]; null: dense, slot j is key j
  const float* softmax_max;        // [batch, n2, s1, n1 / n2]
  const float* softmax_sum;
  float* index_max;                // [rows] dense: index statistics (read when stats_given, else written)
  float* index_sum;
  const int32_t* act_q;     // [batch] or null
  const int32_t* act_k;
  void* d_query_index;      // [rows, g, d_idx]
  void* d_weights;          // [rows, g], dtype_w
  void* d_key_index;        // [batch * s2, d_idx]
  float* loss;              // [1]
  float* di;                // [rows, topk]  scratch, zeroed by the caller: index scores, then dI
  float* p_buf;             // [rows, topk]  scratch, zeroed by the caller: sum over heads of the attention probabilities
  float* loss_parts;        // [rows]        scratch
  float* dki_acc;           // [batch * s2, d_idx] scratch, zeroed by the caller
  int32_t batch, s1, s2, n1, n2, d, d_rope, g, d_idx, topk, dtype_w;
  int32_t stats_given;   // dense: index_max / index_sum come from the caller
  int32_t lse_only;      // dense: stop after the index statistics
  float scale;
};

constexpr int kSliHeads = 16;
constexpr int kSliKeys = 32;
constexpr int kSliTeacherKeys = 64;   // keys per step of the tensor-core scoring kernels (one 8-key tile per warp)
constexpr int kSliThreads = 256;
constexpr int kSliPad = 8;
constexpr float kSliEps = 1e-8f;

__device__ __forceinline__ int32_t sli_row_slots(const SliGradDev& p, int32_t row, int32_t* b_out) {
  const int32_t b = row / p.s1, pos = row - b * p.s1;
  const int32_t aq = p.act_q ? p.act_q[b] : p.s1;
  const int32_t ak = p.act_k ? p.act_k[b] : p.s2;
  *b_out = b;
  if (pos >= aq) return 0;
  const int32_t vis = max(ak - aq + pos + 1, 0);
  if (p.sparse_indices == nullptr) return min(min(vis, ak), p.s2);   // dense: every visible key
  return min(min(p.topk, p.s2), vis);   // :72-74
}

// Key position of slot j of a row: the clipped sparse index (:96), or j itself for the dense operator.
__device__ __forceinline__ int32_t sli_slot_key(const SliGradDev& p, const int32_t* idx_row, int32_t j) {
  return idx_row ? min(max(idx_row[j], 0), p.s2 - 1) : j;
}

__device__ __forceinline__ void store_weight(void* w, int32_t dtype_w, int64_t i, float v) {
  if (dtype_w == DSA_DTYPE_FP32) ((float*)w)[i] = v;
  else if (dtype_w == DSA_DTYPE_FP16) ((__half*)w)[i] = __float2half_rn(v);
  else ((__nv_bfloat16*)w)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float sli_block_reduce(float v, float* red /*[8]*/, bool is_max) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();   // `red` may still be read from an earlier reduction
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < kSliThreads / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

// Stages `heads` rows of width `wa` (+ `wb` from a second tensor) into shared memory, zero past `have`.
template <typename T>
__device__ __forceinline__ void sli_stage_heads(T* dst, int stride, const T* a, int wa, const T* b, int wb, int h0,
                                                int have, int heads = kSliHeads) {
  const int w = wa + wb;
  for (int i = threadIdx.x; i < heads * w; i += kSliThreads) {
    const int h = i / w, c = i - h * w;
    T v = from_f32<T>(0.f);
    if (h0 + h < have) v = c < wa ? a[(int64_t)(h0 + h) * wa + c] : b[(int64_t)(h0 + h) * wb + (c - wa)];
    dst[h * stride + c] = v;
  }
}

// Gathers the rows rows_s[0..nkeys) (16-byte chunks) of one or two key tensors into shared memory
// with cp.async (all of a thread's copies are in flight together; zeros for rows_s[k] < 0) and waits
// for this thread's copies; the caller's barrier makes them visible to the block.
// Row rows_s[k] of a tensor with `nh` heads per position is row rows_s[k] * nh + head.
template <typename T>
__device__ __forceinline__ void sli_gather_keys(T* dst, int stride, const T* a, int wa, const T* b, int wb,
                                                const int64_t* rows_s, int nh = 1, int head = 0,
                                                int nkeys = kSliKeys) {
  const int ca = wa / 8, cb = wb / 8, ct = ca + cb;
  for (int i = threadIdx.x; i < nkeys * ct; i += kSliThreads) {
    const int k = i / ct, c = i - k * ct;
    const int64_t r = rows_s[k] < 0 ? -1 : rows_s[k] * nh + head;
    const T* src = a;
    if (r >= 0) src = c < ca ? a + r * wa + c * 8 : b + r * wb + (c - ca) * 8;
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(&dst[k * stride + c * 8]);
    const int bytes = r >= 0 ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_all;" ::: "memory");
}

// Tensor-core scores (mma.sync m16n8k16, fp32 accumulation) of the 16 staged heads against keys
// n0 .. n0+7 of `ks` over `w` columns (a multiple of 64): out[0..1] = head lane/4, keys n0 + 2 (lane%4)
// (+1); out[2..3] = head lane/4 + 8, same keys.  Rows of `stride` elements (16-byte multiples).
template <typename T>
__device__ __forceinline__ void sli_tile_scores(const T* qs, const T* ks, int stride, int w, int n0, float (&out)[4]) {
  const int lane = threadIdx.x & 31;
  const uint32_t a_addr =
      (uint32_t)__cvta_generic_to_shared(qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * stride + (lane >> 4) * 8);
  const uint32_t b_addr = (uint32_t)__cvta_generic_to_shared(&ks[(n0 + (lane & 7)) * stride + (lane >> 3) * 8]);
  float cs[4][4];
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int e = 0; e < 4; ++e) cs[u][e] = 0.f;
  for (int s = 0; s < w / 16; s += 4) {
    uint32_t a[4][4], b[4][2];
#pragma unroll
    for (int u = 0; u < 4; ++u) ldmatrix_x4(a[u], a_addr + (s + u) * 16 * (int)sizeof(T));
#pragma unroll
    for (int u = 0; u < 4; u += 2) {
      uint32_t r[4];
      ldmatrix_x4(r, b_addr + (s + u) * 16 * (int)sizeof(T));
      b[u][0] = r[0]; b[u][1] = r[1]; b[u + 1][0] = r[2]; b[u + 1][1] = r[3];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) mma_16816<T>(cs[u], a[u], b[u][0], b[u][1]);
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) out[e] = (cs[0][e] + cs[1][e]) + (cs[2][e] + cs[3][e]);
}

// Number of head chunks (of hb heads) of the attention side (per key head) and of the index side.
__host__ __device__ inline int sli_att_chunks(int n1, int n2, int hb = kSliHeads) { return n2 * ((n1 / n2 + hb - 1) / hb); }
__host__ __device__ inline int sli_idx_chunks(int g, int hb = kSliHeads) { return (g + hb - 1) / hb; }

// grid = (rows, attention chunks + index chunks) (index chunks only when lse_only); block = 256.
// MT = 16-head tiles per block (HB = 16 MT heads: two tiles halve the key gathers per row).
// dynamic smem: (HB + 64) * stride elements of T.  A block keeps its HB heads in shared memory,
// walks over the row's keys 64 at a time (each warp scores one tile of 8 keys on the tensor cores)
// and adds its heads' share of p[k] (attention chunks) or of I[k] (index chunks) into the row's fp32
// buffers (zeroed by the caller).
template <typename T, int MT>
__global__ void __launch_bounds__(kSliThreads, 2) sli_teacher_kernel(SliGradDev p, int stride) {
  constexpr int HB = kSliHeads * MT;
  extern __shared__ __align__(16) unsigned char sli_smem[];
  T* qs = reinterpret_cast<T*>(sli_smem);
  T* ks = qs + HB * stride;
  __shared__ int64_t rows_s[kSliTeacherKeys];
  __shared__ float max_s[HB], inv_s[HB], w_s[HB];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int32_t row = blockIdx.x;
  int32_t b;
  const int32_t n = sli_row_slots(p, row, &b);
  if (n == 0) return;
  const bool dense = p.sparse_indices == nullptr;
  const int32_t pos = row - b * p.s1;
  const int32_t* idx_row = dense ? nullptr : p.sparse_indices + (int64_t)row * p.topk;
  const int grp = p.n1 / p.n2;                    // query heads per attention key head
  const int att_chunks = p.lse_only ? 0 : sli_att_chunks(p.n1, p.n2, HB);
  const int ch = blockIdx.y;
  const int phase = ch < att_chunks ? 0 : 1;      // 0: attention distribution p, 1: index scores I
  int kv = 0, h0, h_end;
  if (phase == 0) {
    const int cpk = att_chunks / p.n2;
    kv = ch / cpk;
    h0 = kv * grp + (ch - kv * cpk) * HB;
    h_end = (kv + 1) * grp;
  } else {
    h0 = (ch - att_chunks) * HB;
    h_end = p.g;
  }
  const int w = phase == 0 ? p.d + p.d_rope : p.d_idx;
  float* acc_row = (phase == 0 ? p.p_buf : p.di) + (int64_t)row * p.topk;

  if (phase == 0) {
    const T* q = (const T*)p.query + (int64_t)row * p.n1 * p.d;
    const T* qr = p.d_rope ? (const T*)p.query_rope + (int64_t)row * p.n1 * p.d_rope : nullptr;
    sli_stage_heads<T>(qs, stride, q, p.d, qr, p.d_rope, h0, h_end, HB);
  } else {
    sli_stage_heads<T>(qs, stride, (const T*)p.query_index + (int64_t)row * p.g * p.d_idx, p.d_idx, (const T*)nullptr, 0,
                       h0, h_end, HB);
  }
  if (tid < HB) {
    const int h = h0 + tid;
    if (phase == 0) {
      const int64_t si = (((int64_t)b * p.n2 + kv) * p.s1 + pos) * grp + (h - kv * grp);   // [batch, n2, s1, grp]
      max_s[tid] = h < h_end ? p.softmax_max[si] : 0.f;
      inv_s[tid] = h < h_end ? 1.f / (p.softmax_sum[si] + kSliEps) : 0.f;
    } else {
      w_s[tid] = h < h_end ? load_weight(p.weights, p.dtype_w, (int64_t)row * p.g + h) : 0.f;
    }
  }
  for (int32_t j0 = 0; j0 < n; j0 += kSliTeacherKeys) {
    __syncthreads();   // heads staged; the previous step is done with ks and rows_s
    if (tid < kSliTeacherKeys) {
      const int32_t j = j0 + tid;
      rows_s[tid] = j < n ? (int64_t)b * p.s2 + sli_slot_key(p, idx_row, j) : -1;
    }
    __syncthreads();
    if (phase == 0)
      sli_gather_keys<T>(ks, stride, (const T*)p.key, p.d, (const T*)p.key_rope, p.d_rope, rows_s, p.n2, kv,
                         kSliTeacherKeys);
    else
      sli_gather_keys<T>(ks, stride, (const T*)p.key_index, p.d_idx, (const T*)nullptr, 0, rows_s, 1, 0,
                         kSliTeacherKeys);
    __syncthreads();
    // this thread: heads g and g + 8 of every head tile, keys 2c and 2c + 1 of the warp's key tile;
    // sum over the block's heads
    float t0 = 0.f, t1 = 0.f;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float sc[4];
      sli_tile_scores<T>(qs + mt * kSliHeads * stride, ks, stride, w, warp * 8, sc);
      const int ha = mt * kSliHeads + g, hb = ha + 8;
      if (phase == 0) {
        t0 += expf(sc[0] * p.scale - max_s[ha]) * inv_s[ha] + expf(sc[2] * p.scale - max_s[hb]) * inv_s[hb];
        t1 += expf(sc[1] * p.scale - max_s[ha]) * inv_s[ha] + expf(sc[3] * p.scale - max_s[hb]) * inv_s[hb];
      } else {
        t0 += fmaxf(sc[0], 0.f) * w_s[ha] + fmaxf(sc[2], 0.f) * w_s[hb];
        t1 += fmaxf(sc[1], 0.f) * w_s[ha] + fmaxf(sc[3], 0.f) * w_s[hb];
      }
    }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      t0 += __shfl_xor_sync(0xffffffffu, t0, o);
      t1 += __shfl_xor_sync(0xffffffffu, t1, o);
    }
    if (g == 0) {
      const int32_t j = j0 + warp * 8 + 2 * c;
      if (j < n) atomicAdd(&acc_row[j], t0);
      if (j + 1 < n) atomicAdd(&acc_row[j + 1], t1);
    }
  }
}

// Attention side of the dense operator when a key head serves fewer than 16 query heads (n1 / n2 in
// {1, 2, 4, 8}; multi-head attention is 1).  The rows of a batch walk over the same keys, so a block
// takes 16 / grp consecutive rows times the grp heads of one key head: 16 (row, head) pairs share each
// staged block of 64 keys, where the per-row kernel above would fill only grp of its 16 head slots.
// grid = (batch * ceil(s1 / (16 / grp)), n2); block = 256; dynamic smem as above.
template <typename T>
__global__ void __launch_bounds__(kSliThreads, 2) sli_dense_teacher_kernel(SliGradDev p, int stride) {
  extern __shared__ __align__(16) unsigned char sli_smem[];
  T* qs = reinterpret_cast<T*>(sli_smem);
  T* ks = qs + kSliHeads * stride;
  __shared__ int64_t rows_s[kSliTeacherKeys];
  __shared__ float max_s[kSliHeads], inv_s[kSliHeads];
  __shared__ int32_t n_s[kSliHeads];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = p.n1 / p.n2, rpb = kSliHeads / grp;
  const int blocks_per_batch = (p.s1 + rpb - 1) / rpb;
  const int32_t b = blockIdx.x / blocks_per_batch;
  const int32_t pos0 = (blockIdx.x - b * blocks_per_batch) * rpb;
  const int kv = blockIdx.y;
  const int w = p.d + p.d_rope;

  if (tid < kSliHeads) {
    const int r = tid / grp, hh = tid - r * grp;
    const int32_t pos = pos0 + r;
    int32_t n = 0, bb;
    if (pos < p.s1) n = sli_row_slots(p, b * p.s1 + pos, &bb);
    n_s[tid] = n;
    const int64_t si = (((int64_t)b * p.n2 + kv) * p.s1 + min(pos, p.s1 - 1)) * grp + hh;   // [batch, n2, s1, grp]
    max_s[tid] = n > 0 ? p.softmax_max[si] : 0.f;
    inv_s[tid] = n > 0 ? 1.f / (p.softmax_sum[si] + kSliEps) : 0.f;
  }
  for (int i = tid; i < kSliHeads * w; i += kSliThreads) {
    const int m = i / w, c = i - m * w;
    const int r = m / grp, hh = m - r * grp;
    const int32_t pos = pos0 + r;
    T v = from_f32<T>(0.f);
    if (pos < p.s1) {
      const int64_t qh = ((int64_t)b * p.s1 + pos) * p.n1 + kv * grp + hh;
      v = c < p.d ? ((const T*)p.query)[qh * p.d + c] : ((const T*)p.query_rope)[qh * p.d_rope + (c - p.d)];
    }
    qs[m * stride + c] = v;
  }
  __syncthreads();
  int32_t nmax = 0;
#pragma unroll
  for (int m = 0; m < kSliHeads; ++m) nmax = max(nmax, n_s[m]);
  const int g = lane >> 2, c = lane & 3;
  const int m0 = g, m1 = g + 8;         // this thread's two (row, head) pairs in a score tile
  const int32_t n0 = n_s[m0], n1 = n_s[m1];
  float* acc0 = p.p_buf + ((int64_t)b * p.s1 + pos0 + m0 / grp) * p.topk;
  float* acc1 = p.p_buf + ((int64_t)b * p.s1 + pos0 + m1 / grp) * p.topk;
  for (int32_t j0 = 0; j0 < nmax; j0 += kSliTeacherKeys) {
    __syncthreads();   // the previous step is done with ks and rows_s
    if (tid < kSliTeacherKeys) rows_s[tid] = j0 + tid < nmax ? (int64_t)b * p.s2 + j0 + tid : -1;
    __syncthreads();
    sli_gather_keys<T>(ks, stride, (const T*)p.key, p.d, (const T*)p.key_rope, p.d_rope, rows_s, p.n2, kv,
                       kSliTeacherKeys);
    __syncthreads();
    float sc[4];
    sli_tile_scores<T>(qs, ks, stride, w, warp * 8, sc);
    const int32_t j = j0 + warp * 8 + 2 * c;
    if (j < n0) atomicAdd(&acc0[j], expf(sc[0] * p.scale - max_s[m0]) * inv_s[m0]);
    if (j + 1 < n0) atomicAdd(&acc0[j + 1], expf(sc[1] * p.scale - max_s[m0]) * inv_s[m0]);
    if (j < n1) atomicAdd(&acc1[j], expf(sc[2] * p.scale - max_s[m1]) * inv_s[m1]);
    if (j + 1 < n1) atomicAdd(&acc1[j + 1], expf(sc[3] * p.scale - max_s[m1]) * inv_s[m1]);
  }
}

// grid = rows; block = 256.  Student distribution from the row's index scores, dI = student - p and
// the row's KL term; dI replaces the index scores in place.  With lse_only only the statistics.
__global__ void __launch_bounds__(kSliThreads) sli_student_kernel(SliGradDev p) {
  __shared__ float red8[kSliThreads / 32];
  const int tid = threadIdx.x;
  const int32_t row = blockIdx.x;
  int32_t b;
  const int32_t n = sli_row_slots(p, row, &b);
  const bool dense = p.sparse_indices == nullptr;
  if (n == 0) {
    if (tid == 0) {
      if (!p.lse_only) p.loss_parts[row] = 0.f;
      if (dense && !p.stats_given) { p.index_max[row] = -INFINITY; p.index_sum[row] = 0.f; }
    }
    return;
  }
  float* di = p.di + (int64_t)row * p.topk;       // holds I[k] on entry
  // softmax of the index scores (:95-103), or, for the dense operator, the scores normalised with
  // the index statistics (dense_loss_backward_triton.py:300-312)
  float m, se;
  if (dense && p.stats_given) {
    m = p.index_max[row];
    se = p.index_sum[row];
  } else {
    m = -INFINITY;
    for (int k = tid; k < n; k += kSliThreads) m = fmaxf(m, di[k]);
    m = sli_block_reduce(m, red8, true);
    se = 0.f;
    for (int k = tid; k < n; k += kSliThreads) se += expf(di[k] - m);
    se = sli_block_reduce(se, red8, false);
    if (dense && tid == 0) { p.index_max[row] = m; p.index_sum[row] = se; }
  }
  if (p.lse_only) return;
  if (dense && !(se > 0.f)) {           // the reference skips such rows: no gradient, no loss
    for (int k = tid; k < n; k += kSliThreads) di[k] = 0.f;
    if (tid == 0) p.loss_parts[row] = 0.f;
    return;
  }
  const float* pb = p.p_buf + (int64_t)row * p.topk;
  const float inv = dense ? 1.f / fmaxf(se, kSliEps) : 1.f / (se + kSliEps);
  const float inv_n1 = 1.f / (float)p.n1;
  float kl = 0.f;
  for (int k = tid; k < n; k += kSliThreads) {
    const float si = expf(di[k] - m) * inv, pk = pb[k] * inv_n1;
    di[k] = si - pk;
    const float pc = fmaxf(pk, kSliEps), sc = fmaxf(si, kSliEps);
    kl += pc * (logf(pc) - logf(sc));
  }
  kl = sli_block_reduce(kl, red8, false);
  if (tid == 0) p.loss_parts[row] = kl;
}

// MT = 16-head tiles per block (HB = 16 MT heads; two tiles only for d_idx = 128, where the dQI
// accumulators of both fit in registers: half the steps, gathers and dKI reductions per row).
// grid = (rows, ceil(g / HB)); block = 256.  dynamic smem: (HB + 64) * (d_idx + pad) elements of T.
// Per step of 64 keys, all three products run on the tensor cores (mma.sync m16n8k16): the index
// scores of the block's heads (one 8-key tile per warp and head tile), dQI += ds . ki (each warp owns
// d_idx / 64 column tiles of every head tile, accumulated in registers over the whole row) and
// dKI += ds^T . qi (a warp takes one 16-key tile and half of the columns; its tiles leave as 16-byte
// fp32 reductions).  ds is an fp32 value: it enters the second and third product as a high and a low
// io-dtype part, for fp16 scaled by a power of two per step so that neither part leaves the format's
// range.
template <typename T, int MT>
__global__ void __launch_bounds__(kSliThreads, 2) sli_grad_kernel(SliGradDev p) {
  extern __shared__ __align__(16) unsigned char sli_smem[];
  constexpr int HB = kSliHeads * MT;
  constexpr int NTW = MT == 1 ? 8 : 2;     // most dQI column tiles per warp and head tile
  constexpr int KS = kSliTeacherKeys, PK = KS + 8, PH = HB + 8;
  constexpr bool kScaled = sizeof(T) == 2 && !kIsBf16<T>;
  const int stride = p.d_idx + kSliPad;
  T* qs = reinterpret_cast<T*>(sli_smem);
  T* ks = qs + HB * stride;
  __shared__ __align__(16) T ds_hi[HB * PK], ds_lo[HB * PK];   // [head][key]
  __shared__ __align__(16) T dst_hi[KS * PH], dst_lo[KS * PH]; // [key][head]
  __shared__ float di_s[KS], w_s[HB], red_s[kSliThreads / 32], dw_s[kSliThreads / 32][HB];
  __shared__ int64_t rows_s[KS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int32_t row = blockIdx.x;
  const int32_t h0 = blockIdx.y * HB;
  int32_t b;
  const int32_t n = sli_row_slots(p, row, &b);
  const int ntw = p.d_idx / 64;           // dQI column tiles of this warp: columns 8 (warp * ntw + t) ..
  float acc[MT][NTW][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int t = 0; t < NTW; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][t][e] = 0.f;
  float dw[MT][2];                        // dW partial sums of heads 16 mt + g and + 8
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) dw[mt][0] = dw[mt][1] = 0.f;
  int dq_exp = 127;                       // acc holds dQI * 2^dq_exp (fp16 only)

  if (n > 0) {
    const T* qi = (const T*)p.query_index + (int64_t)row * p.g * p.d_idx;
    sli_stage_heads<T>(qs, stride, qi, p.d_idx, (const T*)nullptr, 0, h0, p.g, HB);
    if (tid < HB) w_s[tid] = h0 + tid < p.g ? load_weight(p.weights, p.dtype_w, (int64_t)row * p.g + h0 + tid) : 0.f;
    const int32_t* idx_row = p.sparse_indices ? p.sparse_indices + (int64_t)row * p.topk : nullptr;
    const float* di = p.di + (int64_t)row * p.topk;
    for (int32_t j0 = 0; j0 < n; j0 += KS) {
      __syncthreads();
      if (tid < KS) {
        const int32_t j = j0 + tid;
        rows_s[tid] = j < n ? (int64_t)b * p.s2 + sli_slot_key(p, idx_row, j) : -1;
        di_s[tid] = j < n ? di[j] : 0.f;
      }
      __syncthreads();
      sli_gather_keys<T>(ks, stride, (const T*)p.key_index, p.d_idx, (const T*)nullptr, 0, rows_s, 1, 0, KS);
      __syncthreads();
      float dsv[MT][4];
      {
        const int k = warp * 8 + 2 * c;
        const float d0 = di_s[k], d1 = di_s[k + 1];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          float sc[4];
          sli_tile_scores<T>(qs + mt * kSliHeads * stride, ks, stride, p.d_idx, warp * 8, sc);
          const float wa = w_s[mt * kSliHeads + g], wb = w_s[mt * kSliHeads + g + 8];
          dw[mt][0] = fmaf(d0, fmaxf(sc[0], 0.f), fmaf(d1, fmaxf(sc[1], 0.f), dw[mt][0]));
          dw[mt][1] = fmaf(d0, fmaxf(sc[2], 0.f), fmaf(d1, fmaxf(sc[3], 0.f), dw[mt][1]));
          dsv[mt][0] = sc[0] > 0.f ? d0 * wa : 0.f;
          dsv[mt][1] = sc[1] > 0.f ? d1 * wa : 0.f;
          dsv[mt][2] = sc[2] > 0.f ? d0 * wb : 0.f;
          dsv[mt][3] = sc[3] > 0.f ? d1 * wb : 0.f;
        }
      }
      float up_k = 1.f, up_q = 1.f, dk_down = 1.f;
      if constexpr (kScaled) {
        float m = 0.f;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) m = fmaxf(m, fabsf(dsv[mt][e]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red_s[warp] = m;
        __syncthreads();
        m = red_s[0];
#pragma unroll
        for (int wv = 1; wv < kSliThreads / 32; ++wv) m = fmaxf(m, red_s[wv]);
        // (a chunk whose values are all zero must not pin the accumulator's scale: it keeps the
        // current one, or 2^100 before the first chunk with a non-zero value)
        int e = (m > 0.f && m < INFINITY) ? 13 - ilogbf(m) : min(dq_exp, 100);
        e = max(-100, min(100, e));
        if (e < dq_exp) {                 // the accumulator follows the smallest scale seen so far
          const float f = scalbnf(1.f, e - dq_exp);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int t = 0; t < NTW; ++t)
#pragma unroll
              for (int x = 0; x < 4; ++x) acc[mt][t][x] *= f;
          dq_exp = e;
        }
        up_k = scalbnf(1.f, e);
        up_q = scalbnf(1.f, dq_exp);
        dk_down = scalbnf(1.f, -e);
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = mt * kSliHeads + g + (e >> 1) * 8, k = warp * 8 + 2 * c + (e & 1);
          const float dk_ = dsv[mt][e] * up_k, dq_ = dsv[mt][e] * up_q;
          const T kh = from_f32<T>(dk_), qh = from_f32<T>(dq_);
          dst_hi[k * PH + h] = kh;
          dst_lo[k * PH + h] = from_f32<T>(dk_ - to_f32<T>(kh));
          ds_hi[h * PK + k] = qh;
          ds_lo[h * PK + k] = from_f32<T>(dq_ - to_f32<T>(qh));
        }
      __syncthreads();

      // dQI += ds . ki : HB heads x (8 ntw) columns per warp, 64 keys deep
#pragma unroll
      for (int k0 = 0; k0 < KS; k0 += 16) {
        uint32_t ah[MT][4], al[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          load_a_frag<T>(ah[mt], ds_hi, PK, mt * kSliHeads, k0);
          load_a_frag<T>(al[mt], ds_lo, PK, mt * kSliHeads, k0);
        }
#pragma unroll
        for (int t = 0; t < NTW; ++t) {
          if (t < ntw) {
            uint32_t b0, b1;
            ldmatrix_b_trans<T>(b0, b1, &ks[k0 * stride + (warp * ntw + t) * 8], stride);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_16816<T>(acc[mt][t], ah[mt], b0, b1);
              mma_16816<T>(acc[mt][t], al[mt], b0, b1);
            }
          }
        }
      }
      // dKI += ds^T . qi : this warp's 16 keys x half of the columns, HB heads deep
      {
        const int kt = warp & 3, nhalf = warp >> 2, nt_half = p.d_idx / 16;
        uint32_t ah[MT][4], al[MT][4];
#pragma unroll
        for (int hs = 0; hs < MT; ++hs) {
          load_a_frag<T>(ah[hs], dst_hi, PH, kt * 16, hs * 16);
          load_a_frag<T>(al[hs], dst_lo, PH, kt * 16, hs * 16);
        }
        const int64_t r_lo = rows_s[kt * 16 + g], r_hi = rows_s[kt * 16 + g + 8];
        for (int t = 0; t < nt_half; ++t) {
          const int n0 = (nhalf * nt_half + t) * 8;
          float cf[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int hs = 0; hs < MT; ++hs) {
            uint32_t b0, b1;
            ldmatrix_b_trans<T>(b0, b1, &qs[hs * 16 * stride + n0], stride);
            mma_16816<T>(cf, ah[hs], b0, b1);
            mma_16816<T>(cf, al[hs], b0, b1);
          }
          if constexpr (kScaled) {
#pragma unroll
            for (int x = 0; x < 4; ++x) cf[x] *= dk_down;
          }
          red_tile(p.dki_acc, p.d_idx, r_lo, r_hi, n0, cf);
        }
      }
    }
  }
  // dW: sum over the four lanes that share a head, then over the warps; dQI of this head chunk
  // (zeros for unused rows)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      dw[mt][u] += __shfl_xor_sync(0xffffffffu, dw[mt][u], 1);
      dw[mt][u] += __shfl_xor_sync(0xffffffffu, dw[mt][u], 2);
    }
  __syncthreads();
  if (c == 0) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      dw_s[warp][mt * kSliHeads + g] = dw[mt][0];
      dw_s[warp][mt * kSliHeads + g + 8] = dw[mt][1];
    }
  }
  __syncthreads();
  if (tid < HB && h0 + tid < p.g) {
    float sum = 0.f;
#pragma unroll
    for (int wv = 0; wv < kSliThreads / 32; ++wv) sum += dw_s[wv][tid];
    store_weight(p.d_weights, p.dtype_w, (int64_t)row * p.g + h0 + tid, sum);
  }
  const float dq_down = kScaled ? scalbnf(1.f, -dq_exp) : 1.f;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int t = 0; t < NTW; ++t) {
      if (t < ntw) {
        const int col = (warp * ntw + t) * 8 + 2 * c;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int h = mt * kSliHeads + g + half * 8;
          if (h0 + h >= p.g) continue;
          T* dst = (T*)p.d_query_index + ((int64_t)row * p.g + h0 + h) * p.d_idx + col;
          dst[0] = from_f32<T>(acc[mt][t][2 * half] * dq_down);
          dst[1] = from_f32<T>(acc[mt][t][2 * half + 1] * dq_down);
        }
      }
    }
}

// Dense softmax statistics from a row-major fp32 score matrix (leading dimension ld) that holds the
// index scores of every visible key of a row, as the indexer's scoring kernels leave them:
// maximum and sum of exponentials over the visible prefix; -inf / 0 for rows that see no key.
// grid = rows; block = 256.
__global__ void __launch_bounds__(kSliThreads) sli_lse_rows_kernel(SliGradDev p, const float* __restrict__ scores,
                                                                   int64_t ld) {
  __shared__ float red8[kSliThreads / 32];
  const int tid = threadIdx.x;
  const int32_t row = blockIdx.x;
  int32_t b;
  const int32_t n = sli_row_slots(p, row, &b);
  if (n == 0) {
    if (tid == 0) { p.index_max[row] = -INFINITY; p.index_sum[row] = 0.f; }
    return;
  }
  const float* s = scores + (int64_t)row * ld;
  float m = -INFINITY;
  for (int k = tid; k < n; k += kSliThreads) m = fmaxf(m, s[k]);
  m = sli_block_reduce(m, red8, true);
  float se = 0.f;
  for (int k = tid; k < n; k += kSliThreads) se += expf(s[k] - m);
  se = sli_block_reduce(se, red8, false);
  if (tid == 0) { p.index_max[row] = m; p.index_sum[row] = se; }
}

// fp32 accumulator -> d_key_index; block 0 also adds up the rows' loss terms in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256) sli_finalize_kernel(SliGradDev p, int64_t total, int32_t rows) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    ((T*)p.d_key_index)[i] = from_f32<T>(p.dki_acc[i]);
  if (blockIdx.x == 0) {
    __shared__ float red[256];
    float s = 0.f;
    for (int r = threadIdx.x; r < rows; r += 256) s += p.loss_parts[r];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
      if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
      __syncthreads();
    }
    if (threadIdx.x == 0) p.loss[0] = red[0];
  }
}

}  // namespace dsa
