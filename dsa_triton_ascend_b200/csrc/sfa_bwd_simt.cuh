// Portable (CUDA-core) sparse flash attention backward: any head count, D in {128,256,512}, BSND and
// TND, token-wise and block-wise indices.  Same math as the reference's backward
// (sparse_flash_attention_grad_triton.py:100-470, golden sparse_flash_attention_grad_numpy.py:96-135):
// the forward statistics rebuild the probabilities,
//     P = exp(score - softmax_max) / softmax_sum,  dP = dO . k_nope,  delta = dO . O,
//     dS = P * (dP - delta) * scale,
// d_query / d_query_rope are per query row, d_key / d_key_rope / d_value are scatter-added over the
// rows that selected a key.  Where the reference keeps dS and P in an io-dtype workspace between two
// passes and converts fp32 scatter buffers afterwards, one kernel here does both products per chunk
// of gathered keys with P and dS in fp32 shared memory, adds into fp32 accumulators with 16-byte
// vector reductions, and a second small kernel rounds the accumulators to the io dtype.
#pragma once

#include "dsa_common.cuh"
#include "sfa_fwd_mma.cuh"

namespace dsa {

struct SfaGradDev {
  SeqDesc seq;
  const void* query;
  const void* query_rope;
  const void* key;
  const void* key_rope;
  const int32_t* sparse_indices;
  const void* d_out;
  const void* out;
  const float* softmax_max;
  const float* softmax_sum;
  void* d_query;
  void* d_query_rope;
  float* dk_acc;  // [key_rows, d + d_rope]  QK path (nope | rope)
  float* dv_acc;  // [key_rows, d]           PV path
  int32_t rows, n1, d, d_rope;
  int32_t sparse_count, sparse_block_size;
  float scale;
};

constexpr int kSfaGradHeads = 16;   // heads per block
constexpr int kSfaGradKeys = 32;    // gathered keys per step
constexpr int kSfaGradThreads = 256;
constexpr int kSfaGradPad = 8;      // elements of row padding (16-byte loads stay conflict free)

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

inline size_t sfa_grad_smem_bytes(int d, int d_rope, size_t elem) {
  return ((size_t)(kSfaGradHeads + kSfaGradKeys) * (d + d_rope + kSfaGradPad) +
          (size_t)kSfaGradHeads * (d + kSfaGradPad)) * elem;
}

// grid = (rows, ceil(n1 / 16)); block = 256 threads.
// dynamic smem: q [16][d+dr+pad] | keys [32][d+dr+pad] | dO [16][d+pad], elements of T.
template <typename T>
__global__ void __launch_bounds__(kSfaGradThreads) sfa_bwd_simt_kernel(SfaGradDev p) {
  extern __shared__ __align__(16) unsigned char sfa_grad_smem[];
  const int32_t dq = p.d + p.d_rope;
  const int32_t stride = dq + kSfaGradPad;
  const int32_t dstride = p.d + kSfaGradPad;
  T* qs = reinterpret_cast<T*>(sfa_grad_smem);
  T* ks = qs + kSfaGradHeads * stride;
  T* dos = ks + kSfaGradKeys * stride;
  __shared__ float ps[kSfaGradHeads][kSfaGradKeys + 1];
  __shared__ float dss[kSfaGradHeads][kSfaGradKeys + 1];
  __shared__ float delta_s[kSfaGradHeads], max_s[kSfaGradHeads], sum_s[kSfaGradHeads];
  __shared__ int32_t tok_s[kSfaGradKeys];
  __shared__ int64_t krow_s[kSfaGradKeys];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t row = blockIdx.x;
  const int32_t h0 = blockIdx.y * kSfaGradHeads;
  const RowInfo ri = row_info(p.seq, row);
  const bool row_active = ri.pos < ri.act_q && ri.threshold > 0 && ri.act_k > 0;

  // d_query accumulator: head = tid / 16, columns 2*(tid%16) + 32*j (+1) of nope|rope
  const int ah = tid >> 4, ac = (tid & 15) * 2;
  float acc[36];
#pragma unroll
  for (int j = 0; j < 36; ++j) acc[j] = 0.f;

  T* dqn = (T*)p.d_query + ((int64_t)row * p.n1 + h0) * p.d;
  T* dqr = (T*)p.d_query_rope + ((int64_t)row * p.n1 + h0) * p.d_rope;

  if (row_active) {
    // stage q (nope | rope) and dO of the head chunk, zero for heads past n1
    const T* qn = (const T*)p.query + (int64_t)row * p.n1 * p.d;
    const T* qr = (const T*)p.query_rope + (int64_t)row * p.n1 * p.d_rope;
    const T* dout = (const T*)p.d_out + (int64_t)row * p.n1 * p.d;
    for (int i = tid; i < kSfaGradHeads * dq; i += kSfaGradThreads) {
      int h = i / dq, c = i - h * dq;
      T v = from_f32<T>(0.f);
      if (h0 + h < p.n1) v = c < p.d ? qn[(int64_t)(h0 + h) * p.d + c] : qr[(int64_t)(h0 + h) * p.d_rope + (c - p.d)];
      qs[h * stride + c] = v;
    }
    for (int i = tid; i < kSfaGradHeads * p.d; i += kSfaGradThreads) {
      int h = i / p.d, c = i - h * p.d;
      dos[h * dstride + c] = h0 + h < p.n1 ? dout[(int64_t)(h0 + h) * p.d + c] : from_f32<T>(0.f);
    }
    // delta = dO . O per head (16 threads per head), and the forward statistics
    {
      float part = 0.f;
      if (h0 + ah < p.n1) {
        const T* o = (const T*)p.out + ((int64_t)row * p.n1 + h0 + ah) * p.d;
        const T* g = dout + (int64_t)(h0 + ah) * p.d;
        for (int c = tid & 15; c < p.d; c += 16) part = fmaf(to_f32<T>(g[c]), to_f32<T>(o[c]), part);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if ((tid & 15) == 0) {
        const bool hv = h0 + ah < p.n1;
        delta_s[ah] = part;
        max_s[ah] = hv ? p.softmax_max[(int64_t)row * p.n1 + h0 + ah] : 0.f;
        sum_s[ah] = hv ? p.softmax_sum[(int64_t)row * p.n1 + h0 + ah] : 0.f;
      }
    }
  }
  __syncthreads();

  const int32_t* idx_row = p.sparse_indices + (int64_t)row * p.sparse_count;
  const int32_t slots = row_active ? p.sparse_count * p.sparse_block_size : 0;
  const T* kn = (const T*)p.key;
  const T* kr = (const T*)p.key_rope;
  const int nq = dq / 32;              // accumulator column pairs per thread
  const int gk = dq / 4, gv = p.d / 4; // 4-column groups of the two scatter targets

  for (int32_t j0 = 0; j0 < slots; j0 += kSfaGradKeys) {
    int any = 0;
    if (tid < kSfaGradKeys) {
      int32_t j = j0 + tid;
      int32_t tok = j < slots ? sfa_slot_token(p.seq, p.sparse_block_size, ri, idx_row, j) : -1;
      int64_t r = tok >= 0 ? key_row(p.seq, ri, tok) : -1;
      tok_s[tid] = r >= 0 ? tok : -1;
      krow_s[tid] = r;
      any = r >= 0;
    }
    if (!__syncthreads_or(any)) continue;

    // gather the rows (16-byte chunks)
    {
      const int cn = p.d / 8, cr = p.d_rope / 8, ct = cn + cr;
      for (int i = tid; i < kSfaGradKeys * ct; i += kSfaGradThreads) {
        int k = i / ct, c = i - k * ct;
        int64_t kr_ = krow_s[k];
        uint4 v = make_uint4(0, 0, 0, 0);
        if (kr_ >= 0) {
          v = c < cn ? reinterpret_cast<const uint4*>(kn + kr_ * p.d)[c]
                     : reinterpret_cast<const uint4*>(kr + kr_ * p.d_rope)[c - cn];
        }
        *reinterpret_cast<uint4*>(&ks[k * stride + c * 8]) = v;
      }
    }
    __syncthreads();

    // scores and dP: thread -> key = lane, heads warp and warp + 8
    {
      float s0 = 0.f, s1 = 0.f, g0 = 0.f, g1 = 0.f;
      const uint4* kp = reinterpret_cast<const uint4*>(&ks[lane * stride]);
      const uint4* q0 = reinterpret_cast<const uint4*>(&qs[warp * stride]);
      const uint4* q1 = reinterpret_cast<const uint4*>(&qs[(warp + 8) * stride]);
      const uint4* d0 = reinterpret_cast<const uint4*>(&dos[warp * dstride]);
      const uint4* d1 = reinterpret_cast<const uint4*>(&dos[(warp + 8) * dstride]);
      const int cn = p.d / 8;
      for (int c = 0; c < dq / 8; ++c) {
        uint4 kv = kp[c], a = q0[c], b = q1[c];
        const T* kk = reinterpret_cast<const T*>(&kv);
        const T* aa = reinterpret_cast<const T*>(&a);
        const T* bb = reinterpret_cast<const T*>(&b);
        float kf[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          kf[e] = to_f32<T>(kk[e]);
          s0 = fmaf(kf[e], to_f32<T>(aa[e]), s0);
          s1 = fmaf(kf[e], to_f32<T>(bb[e]), s1);
        }
        if (c < cn) {
          uint4 x = d0[c], y = d1[c];
          const T* xx = reinterpret_cast<const T*>(&x);
          const T* yy = reinterpret_cast<const T*>(&y);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            g0 = fmaf(kf[e], to_f32<T>(xx[e]), g0);
            g1 = fmaf(kf[e], to_f32<T>(yy[e]), g1);
          }
        }
      }
      const bool valid = tok_s[lane] >= 0;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int h = warp + half * 8;
        const float sv = (half ? s1 : s0) * p.scale;
        const float gvv = half ? g1 : g0;
        const float l = sum_s[h];
        const float pv = (valid && l > 0.f) ? expf(sv - max_s[h]) / l : 0.f;
        ps[h][lane] = pv;
        dss[h][lane] = pv * (gvv - delta_s[h]) * p.scale;
      }
    }
    __syncthreads();

    // d_query (nope | rope) += dS . k
    for (int k = 0; k < kSfaGradKeys; ++k) {
      const float w = dss[ah][k];
      if (w == 0.f) continue;
      const T* kr_ = &ks[k * stride + ac];
#pragma unroll
      for (int j = 0; j < 18; ++j) {
        if (j < nq) {
          acc[2 * j] = fmaf(w, to_f32<T>(kr_[32 * j]), acc[2 * j]);
          acc[2 * j + 1] = fmaf(w, to_f32<T>(kr_[32 * j + 1]), acc[2 * j + 1]);
        }
      }
    }

    // d_key (nope | rope) += dS^T . q,  d_value += P^T . dO : one unit = 4 columns of one key,
    // summed over the 16 heads of this block, added to the fp32 accumulators in one reduction
    for (int u = tid; u < kSfaGradKeys * (gk + gv); u += kSfaGradThreads) {
      const int k = u / (gk + gv);
      int g = u - k * (gk + gv);
      const int64_t kr_ = krow_s[k];
      if (kr_ < 0) continue;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      if (g < gk) {
#pragma unroll 4
        for (int h = 0; h < kSfaGradHeads; ++h) {
          const float w = dss[h][k];
          const uint2 v = *reinterpret_cast<const uint2*>(&qs[h * stride + 4 * g]);
          const T* e = reinterpret_cast<const T*>(&v);
          a0 = fmaf(w, to_f32<T>(e[0]), a0); a1 = fmaf(w, to_f32<T>(e[1]), a1);
          a2 = fmaf(w, to_f32<T>(e[2]), a2); a3 = fmaf(w, to_f32<T>(e[3]), a3);
        }
        red_add_v4(p.dk_acc + kr_ * dq + 4 * g, a0, a1, a2, a3);
      } else {
        g -= gk;
#pragma unroll 4
        for (int h = 0; h < kSfaGradHeads; ++h) {
          const float w = ps[h][k];
          const uint2 v = *reinterpret_cast<const uint2*>(&dos[h * dstride + 4 * g]);
          const T* e = reinterpret_cast<const T*>(&v);
          a0 = fmaf(w, to_f32<T>(e[0]), a0); a1 = fmaf(w, to_f32<T>(e[1]), a1);
          a2 = fmaf(w, to_f32<T>(e[2]), a2); a3 = fmaf(w, to_f32<T>(e[3]), a3);
        }
        red_add_v4(p.dv_acc + kr_ * p.d + 4 * g, a0, a1, a2, a3);
      }
    }
    __syncthreads();
  }

  // d_query / d_query_rope of this head chunk (zeros for inactive rows)
  if (h0 + ah < p.n1) {
#pragma unroll
    for (int j = 0; j < 18; ++j) {
      if (j < nq) {
        const int c = ac + 32 * j;
        T* dst = c < p.d ? dqn + (int64_t)ah * p.d + c : dqr + (int64_t)ah * p.d_rope + (c - p.d);
        dst[0] = from_f32<T>(acc[2 * j]);
        dst[1] = from_f32<T>(acc[2 * j + 1]);
      }
    }
  }
}

// fp32 accumulators -> d_key [key_rows, d], d_key_rope [key_rows, d_rope], d_value [key_rows, d]
template <typename T>
__global__ void __launch_bounds__(256) sfa_bwd_finalize_kernel(const float* __restrict__ dk_acc,
                                                               const float* __restrict__ dv_acc, T* d_key,
                                                               T* d_key_rope, T* d_value, int64_t key_rows, int32_t d,
                                                               int32_t d_rope) {
  const int32_t dq = d + d_rope, w = dq + d;
  const int64_t total = key_rows * w;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / w;
    const int32_t c = (int32_t)(i - r * w);
    if (c < d) d_key[r * d + c] = from_f32<T>(dk_acc[r * dq + c]);
    else if (c < dq) d_key_rope[r * d_rope + (c - d)] = from_f32<T>(dk_acc[r * dq + c]);
    else d_value[r * d + (c - dq)] = from_f32<T>(dv_acc[r * d + (c - dq)]);
  }
}

}  // namespace dsa
