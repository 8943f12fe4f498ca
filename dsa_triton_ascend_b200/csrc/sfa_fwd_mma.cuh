// Any-shape sparse flash attention forward: any head count, D in {128,256,512}, all layouts,
// token-wise and block-wise indices.  Same math as _sfa_kernel's chunked path
// (sparse_flash_attention_triton.py:461-604): rows gathered by index, invalid slots masked to
// -inf, online softmax with fp32 statistics, probabilities rounded to the io dtype before the
// second product (:520), value = key[..., :D].  One block per (query row, 16 heads) walks over the
// row's slots 32 at a time; both products of a step run on the warp-level tensor-core instructions
// (mma.sync m16n8k16, fp32 accumulation), the softmax in fp32 on the CUDA cores.
#pragma once

#include "dsa_common.cuh"
#include "mma_sync.cuh"

namespace dsa {

struct SfaDev {
  SeqDesc seq;
  const void* query;
  const void* query_rope;
  const void* key;
  const void* key_rope;
  const int32_t* sparse_indices;
  void* out;
  float* softmax_max;
  float* softmax_sum;
  int32_t rows, n1, d, d_rope;
  int32_t sparse_count, sparse_block_size, return_lse;
  float scale;
};

constexpr int kSfaSimtHeads = 16;   // heads per block
constexpr int kSfaSimtKeys = 32;    // gathered keys per step
constexpr int kSfaSimtThreads = 256;
constexpr int kSfaSimtPad = 8;      // elements of row padding (keeps 16-byte loads conflict free)

// Validity and physical row of slot j of a query row (sparse_flash_attention_triton.py:465,
// 1036-1051): returns the logical token or -1.
__device__ __forceinline__ int32_t sfa_slot_token(const SeqDesc& seq, int32_t bs, const RowInfo& ri,
                                                  const int32_t* idx_row, int32_t j) {
  const int32_t id = idx_row[j / bs];
  if (id < 0) return -1;
  const int64_t tok = (int64_t)id * bs + (j % bs);
  if (tok >= ri.threshold || tok >= ri.act_k) return -1;
  if (seq.layout_k != DSA_LAYOUT_PA_BSND && tok >= seq.s2) return -1;
  return (int32_t)tok;
}
__device__ __forceinline__ int32_t sfa_slot_token(const SfaDev& p, const RowInfo& ri, const int32_t* idx_row,
                                                  int32_t j) {
  return sfa_slot_token(p.seq, p.sparse_block_size, ri, idx_row, j);
}

// One query row, 16 heads starting at h0, by one block of 256 threads.
// dynamic smem: (16 + 32) * (d + d_rope + pad) elements of T.
template <typename T>
__device__ __forceinline__ void sfa_fwd_mma_row(const SfaDev& p, int32_t row, int32_t h0) {
  extern __shared__ __align__(16) unsigned char sfa_smem[];
  const int32_t dq = p.d + p.d_rope;
  const int32_t stride = dq + kSfaSimtPad;
  T* qs = reinterpret_cast<T*>(sfa_smem);
  T* ks = qs + kSfaSimtHeads * stride;
  __shared__ float sp[2][kSfaSimtHeads][kSfaSimtKeys + 1];            // partial scores of the two column halves
  __shared__ __align__(16) T pt[kSfaSimtHeads * (kSfaSimtKeys + 8)];  // probabilities as the io dtype, [head][key]
  __shared__ float alpha_s[kSfaSimtHeads];
  __shared__ float l_s[kSfaSimtHeads];
  __shared__ float m_s[kSfaSimtHeads];
  __shared__ int32_t tok_s[kSfaSimtKeys];
  __shared__ int64_t krow_s[kSfaSimtKeys];

  constexpr int PK = kSfaSimtKeys + 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c4 = lane & 3;
  const RowInfo ri = row_info(p.seq, row);
  const bool row_active = ri.pos < ri.act_q && ri.threshold > 0 && ri.act_k > 0;

  // output accumulator: heads g and g + 8, d / 64 column tiles of 8 per warp (warp w: columns
  // (d / 8) w .. (d / 8) (w + 1) - 1), in the mma accumulator layout
  const int ntw = p.d / 64;
  float acc[8][4];
#pragma unroll
  for (int t = 0; t < 8; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

  T* outp = (T*)p.out + ((int64_t)row * p.n1 + h0) * p.d;
  if (!row_active) {
    for (int i = tid; i < kSfaSimtHeads * p.d; i += kSfaSimtThreads) {
      int h = i / p.d;
      if (h0 + h < p.n1) outp[i] = from_f32<T>(0.f);
    }
    if (p.return_lse && tid < kSfaSimtHeads && h0 + tid < p.n1) {
      p.softmax_max[(int64_t)row * p.n1 + h0 + tid] = 0.f;
      p.softmax_sum[(int64_t)row * p.n1 + h0 + tid] = 0.f;
    }
    return;
  }

  // stage the head chunk of q (nope | rope) into shared memory, zero for heads past n1
  {
    const T* qn = (const T*)p.query + (int64_t)row * p.n1 * p.d;
    const T* qr = (const T*)p.query_rope + (int64_t)row * p.n1 * p.d_rope;
    for (int i = tid; i < kSfaSimtHeads * dq; i += kSfaSimtThreads) {
      int h = i / dq, c = i - h * dq;
      T v = from_f32<T>(0.f);
      if (h0 + h < p.n1) v = c < p.d ? qn[(int64_t)(h0 + h) * p.d + c] : qr[(int64_t)(h0 + h) * p.d_rope + (c - p.d)];
      qs[h * stride + c] = v;
    }
  }
  if (tid < kSfaSimtHeads) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
  __syncthreads();

  const int32_t* idx_row = p.sparse_indices + (int64_t)row * p.sparse_count;
  const int32_t slots = p.sparse_count * p.sparse_block_size;
  const T* kn = (const T*)p.key;
  const T* kr = (const T*)p.key_rope;

  // Up to 128 valid slots the softmax is normalised before the probabilities are rounded, which is the
  // order of the golden and of the reference's single-block path (:419-436): pass 0 finds max and
  // sum, pass 1 accumulates.  Longer rows use the online form in one pass.
  __shared__ int32_t nvalid_s;
  if (tid == 0) nvalid_s = 0;
  __syncthreads();
  {
    int32_t part = 0;
    for (int32_t j = tid; j < slots; j += kSfaSimtThreads) part += sfa_slot_token(p, ri, idx_row, j) >= 0;
    if (part) atomicAdd(&nvalid_s, part);
  }
  __syncthreads();
  const bool two_pass = nvalid_s <= 128;
  const int npass = two_pass ? 2 : 1;
  for (int pass = 0; pass < npass; ++pass)
  for (int32_t j0 = 0; j0 < slots; j0 += kSfaSimtKeys) {
    int any = 0;
    if (tid < kSfaSimtKeys) {
      int32_t j = j0 + tid;
      int32_t tok = j < slots ? sfa_slot_token(p, ri, idx_row, j) : -1;
      tok_s[tid] = tok;
      krow_s[tid] = tok >= 0 ? key_row(p.seq, ri, tok) : -1;
      any = tok >= 0;
    }
    if (!__syncthreads_or(any)) continue;

    // gather the rows with cp.async (16-byte chunks, all of a thread's copies in flight together;
    // slots without a key and absent paged blocks are zero-filled, like the un-paged cache)
    {
      const int cn = p.d / 8, cr = p.d_rope / 8, ct = cn + cr;
      for (int i = tid; i < kSfaSimtKeys * ct; i += kSfaSimtThreads) {
        const int k = i / ct, c = i - k * ct;
        const int64_t kr_ = krow_s[k];
        const T* src = kn;
        if (kr_ >= 0) src = c < cn ? kn + kr_ * p.d + c * 8 : kr + kr_ * p.d_rope + (c - cn) * 8;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&ks[k * stride + c * 8]);
        const int bytes = kr_ >= 0 ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_all;" ::: "memory");
    }
    __syncthreads();

    // scores on the tensor cores: warp w takes the 8-key tile w % 4 over half w / 4 of the columns
    {
      const int n0 = (warp & 3) * 8, half = warp >> 2, kh = dq / 32;      // kh 16-column steps per half (even)
      const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(
          qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * stride + (lane >> 4) * 8);
      const uint32_t b_addr = (uint32_t)__cvta_generic_to_shared(&ks[(n0 + (lane & 7)) * stride + (lane >> 3) * 8]);
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
      for (int st = half * kh; st < (half + 1) * kh; st += 2) {
        uint32_t a0[4], a1[4], b[4];
        ldmatrix_x4(a0, a_addr + st * 16 * (int)sizeof(T));
        ldmatrix_x4(a1, a_addr + (st + 1) * 16 * (int)sizeof(T));
        ldmatrix_x4(b, b_addr + st * 16 * (int)sizeof(T));
        mma_16816<T>(c0, a0, b[0], b[1]);
        mma_16816<T>(c1, a1, b[2], b[3]);
      }
      sp[half][g][n0 + 2 * c4] = c0[0] + c1[0];
      sp[half][g][n0 + 2 * c4 + 1] = c0[1] + c1[1];
      sp[half][g + 8][n0 + 2 * c4] = c0[2] + c1[2];
      sp[half][g + 8][n0 + 2 * c4 + 1] = c0[3] + c1[3];
    }
    __syncthreads();

    // softmax step: thread -> key = lane, heads warp and warp + 8
    {
      float s0 = sp[0][warp][lane] + sp[1][warp][lane];
      float s1 = sp[0][warp + 8][lane] + sp[1][warp + 8][lane];
      const bool valid = tok_s[lane] >= 0;
      s0 = valid ? s0 * p.scale : -INFINITY;
      s1 = valid ? s1 * p.scale : -INFINITY;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int h = warp + half * 8;
        float sv = half ? s1 : s0;
        float mx = sv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_old = m_s[h];
        if (two_pass && pass == 1) {
          const float l = l_s[h];
          const float pv = (valid && l > 0.f) ? expf(sv - m_old) / l : 0.f;
          pt[h * PK + lane] = from_f32<T>(pv);
          if (lane == 0) alpha_s[h] = 1.f;
          continue;
        }
        const float m_new = fmaxf(m_old, mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        float pv = valid ? expf(sv - m_safe) : 0.f;
        float sum = pv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        pt[h * PK + lane] = from_f32<T>(pv);
        __syncwarp();
        if (lane == 0) {
          const float a = m_old == -INFINITY ? 0.f : expf(m_old - m_safe);
          alpha_s[h] = a;
          l_s[h] = l_s[h] * a + sum;
          m_s[h] = m_new;
        }
      }
    }
    __syncthreads();

    // accumulate: acc = acc * alpha + P . V   (skipped in the statistics pass)
    if (!(two_pass && pass == 0)) {
      const float a_lo = alpha_s[g], a_hi = alpha_s[g + 8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t < ntw) { acc[t][0] *= a_lo; acc[t][1] *= a_lo; acc[t][2] *= a_hi; acc[t][3] *= a_hi; }
      }
#pragma unroll
      for (int k0 = 0; k0 < kSfaSimtKeys; k0 += 16) {
        uint32_t a[4];
        load_a_frag<T>(a, pt, PK, 0, k0);
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          if (t < ntw) {
            uint32_t b0, b1;
            ldmatrix_b_trans<T>(b0, b1, &ks[k0 * stride + (warp * ntw + t) * 8], stride);
            mma_16816<T>(acc[t], a, b0, b1);
          }
        }
      }
    }
    __syncthreads();
  }

  // epilogue
  {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int h = g + half * 8;
      if (h0 + h >= p.n1) continue;
      const float l = l_s[h];
      const float inv = two_pass ? 1.f : (l > 0.f ? 1.f / l : 0.f);
      T* o = outp + (int64_t)h * p.d;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t < ntw) {
          const int col = (warp * ntw + t) * 8 + 2 * c4;
          o[col] = from_f32<T>(acc[t][2 * half] * inv);
          o[col + 1] = from_f32<T>(acc[t][2 * half + 1] * inv);
        }
      }
    }
    if (p.return_lse && tid < kSfaSimtHeads && h0 + tid < p.n1) {
      const float lt = l_s[tid];
      p.softmax_max[(int64_t)row * p.n1 + h0 + tid] = lt > 0.f ? m_s[tid] : 0.f;
      p.softmax_sum[(int64_t)row * p.n1 + h0 + tid] = lt > 0.f ? lt : 0.f;
    }
  }
}

// grid = (rows, ceil(n1 / 16)); block = 256 threads.
template <typename T>
__global__ void __launch_bounds__(kSfaSimtThreads) sfa_fwd_mma_kernel(SfaDev p) {
  sfa_fwd_mma_row<T>(p, (int32_t)blockIdx.x, (int32_t)blockIdx.y * kSfaSimtHeads);
}

// Recomputes the rows listed in redo_list[0 .. *redo_count) (rows whose scores outgrew the
// tensor-core kernel's fixed reference maximum; normally none, and then every block leaves after
// one load).  Any grid; blocks walk over (listed row, head chunk) pairs.
template <typename T>
__global__ void __launch_bounds__(kSfaSimtThreads) sfa_redo_kernel(SfaDev p, const int32_t* __restrict__ redo_list,
                                                                   const int32_t* __restrict__ redo_count) {
  const int32_t chunks = (p.n1 + kSfaSimtHeads - 1) / kSfaSimtHeads;
  const int64_t work = (int64_t)min(*redo_count, p.rows) * chunks;
  for (int64_t i = blockIdx.x; i < work; i += gridDim.x) {
    __syncthreads();   // the previous row's shared state is no longer read
    sfa_fwd_mma_row<T>(p, redo_list[i / chunks], (int32_t)(i % chunks) * kSfaSimtHeads);
  }
}

}  // namespace dsa
