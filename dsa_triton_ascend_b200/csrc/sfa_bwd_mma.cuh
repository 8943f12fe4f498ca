// Sparse flash attention backward with the five contractions of a key chunk on the warp-level
// tensor-core instructions (mma.sync m16n8k16, fp32 accumulation), for D in {128, 256, 512} and
// D_rope = 64.  Same math as sfa_bwd_simt_kernel (sparse_flash_attention_grad_triton.py:100-470, golden
// sparse_flash_attention_grad_numpy.py:96-135): one block per (query row, 16 or 32 heads) walks over
// the row's selected keys 32 at a time,
//     S  = q . k^T (D + 64 columns)       dP = dO . k_nope^T (D columns)
//     P  = exp(S * scale - max) / sum     dS = P * (dP - delta) * scale
//     dQ += dS . k        dK += dS^T . q        dV += P^T . dO
// q, k and dO are multiplied as the io dtype they arrive in (exact products, fp32 sums).  P and dS
// are fp32 values: each is split into a high and a low io-dtype part (x = hi + lo up to 2^-16
// relative for bf16, 2^-22 for fp16; fp16 parts are scaled per key chunk, see the kernel) and every
// product with them runs twice, so the result carries fp32-like precision where the reference
// rounds P and dS to the io dtype once.  dK / dV leave the block as 16-byte fp32 reductions into the
// accumulators that sfa_bwd_finalize_kernel rounds.
#pragma once

#include "mma_sync.cuh"
#include "sfa_bwd_simt.cuh"

namespace dsa {

constexpr int kSfaMmaDr = 64;
constexpr int kSfaMmaPk = kSfaGradKeys + 8;               // [head][key] operand rows (40 elements)

// Adds the 16 x 8 accumulator tile (rows -> key rows krow_lo / krow_hi of this lane's two rows,
// columns col0 .. col0+7 of a row of `width` floats) into `acc`: lanes pair up so that each issues
// one 16-byte reduction.
__device__ __forceinline__ void red_tile(float* acc, int width, int64_t krow_lo, int64_t krow_hi, int col0,
                                         const float (&c)[4]) {
  const int lane = threadIdx.x & 31, cc = lane & 3;
  const bool odd = lane & 1;
  const float s0 = odd ? c[0] : c[2], s1 = odd ? c[1] : c[3];
  const float r0 = __shfl_xor_sync(0xffffffffu, s0, 1), r1 = __shfl_xor_sync(0xffffffffu, s1, 1);
  const int col = col0 + 2 * (cc & ~1);
  if (!odd) {
    if (krow_lo >= 0) red_add_v4(acc + krow_lo * width + col, c[0], c[1], r0, r1);
  } else {
    if (krow_hi >= 0) red_add_v4(acc + krow_hi * width + col, r0, r1, c[2], c[3]);
  }
}

// MT = 16-head tiles per block (1 or 2): HB = 16 MT heads, 256 MT threads.  Every scatter-add of d_key /
// d_value covers the block's heads, so two tiles halve the reductions per query row; they cost one
// block per SM instead of two (with the same number of warps).
// grid = (rows, ceil(n1 / HB)).  dynamic smem: q [HB][D+72] | keys [32][D+72] | dO [HB][D+8], elements of T.
template <int MT, int D>
inline size_t sfa_grad_mma_smem_bytes(size_t elem) {
  return ((size_t)(16 * MT + kSfaGradKeys) * (D + kSfaMmaDr + kSfaGradPad) + (size_t)16 * MT * (D + kSfaGradPad)) * elem;
}

template <typename T, int MT, int D>
__global__ void __launch_bounds__(256 * MT, MT == 1 ? 2 : 1) sfa_bwd_mma_kernel(SfaGradDev p) {
  constexpr int kSfaMmaD = D, kSfaMmaDq = D + kSfaMmaDr;
  constexpr int kSfaMmaStride = kSfaMmaDq + kSfaGradPad;    // q / key rows, elements
  constexpr int kSfaMmaDStride = kSfaMmaD + kSfaGradPad;    // dO rows
  constexpr int QT = kSfaMmaDq / 64;                        // d_query / d_key column tiles of 8 per warp (9 at D = 512)
  constexpr int VT = kSfaMmaD / 64;                         // d_value column tiles per warp
  constexpr int HB = 16 * MT, NT = 256 * MT;
  constexpr int PH = HB + 8;              // [key][head] operand rows, elements
  extern __shared__ __align__(16) unsigned char sfa_grad_smem[];
  T* qs = reinterpret_cast<T*>(sfa_grad_smem);
  T* ks = qs + HB * kSfaMmaStride;
  T* dos = ks + kSfaGradKeys * kSfaMmaStride;
  __shared__ float ps_f[HB][kSfaGradKeys + 1];
  __shared__ float dp_f[HB][kSfaGradKeys + 1];
  __shared__ __align__(16) T ds_hi[HB * kSfaMmaPk], ds_lo[HB * kSfaMmaPk];         // [head][key]
  __shared__ __align__(16) T dst_hi[kSfaGradKeys * PH], dst_lo[kSfaGradKeys * PH]; // [key][head]
  __shared__ __align__(16) T pt_hi[kSfaGradKeys * PH], pt_lo[kSfaGradKeys * PH];   // [key][head]
  __shared__ float delta_s[HB], max_s[HB], sum_s[HB];
  __shared__ float red_s[NT / 32];
  __shared__ int32_t tok_s[2][kSfaGradKeys];
  __shared__ int64_t krow_s[2][kSfaGradKeys];

  constexpr bool kScaled = sizeof(T) == 2 && !kIsBf16<T>;   // fp16: operands of the second products are scaled
  int dq_exp = 127;                                         // acc holds d_query * 2^dq_exp (fp16 only)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int32_t row = blockIdx.x;
  const int32_t h0 = blockIdx.y * HB;
  const RowInfo ri = row_info(p.seq, row);
  const bool row_active = ri.pos < ri.act_q && ri.threshold > 0 && ri.act_k > 0;
  const int qm0 = (warp >> 3) * 16;       // head tile of this warp in the d_query product
  const int qn0 = (warp & 7) * (QT * 8);  // its first column there and in the d_key product

  // d_query accumulator: 16 heads x 8 QT columns per warp
  float acc[QT][4];
#pragma unroll
  for (int t = 0; t < QT; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

  if (row_active) {
    const T* qn = (const T*)p.query + (int64_t)row * p.n1 * kSfaMmaD;
    const T* qr = (const T*)p.query_rope + (int64_t)row * p.n1 * kSfaMmaDr;
    const T* dout = (const T*)p.d_out + (int64_t)row * p.n1 * kSfaMmaD;
    for (int i = tid; i < HB * (kSfaMmaDq / 8); i += NT) {
      const int h = i / (kSfaMmaDq / 8), ch = i - h * (kSfaMmaDq / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h0 + h < p.n1)
        v = ch < kSfaMmaD / 8 ? reinterpret_cast<const uint4*>(qn + (int64_t)(h0 + h) * kSfaMmaD)[ch]
                              : reinterpret_cast<const uint4*>(qr + (int64_t)(h0 + h) * kSfaMmaDr)[ch - kSfaMmaD / 8];
      *reinterpret_cast<uint4*>(&qs[h * kSfaMmaStride + ch * 8]) = v;
    }
    for (int i = tid; i < HB * (kSfaMmaD / 8); i += NT) {
      const int h = i / (kSfaMmaD / 8), ch = i - h * (kSfaMmaD / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h0 + h < p.n1) v = reinterpret_cast<const uint4*>(dout + (int64_t)(h0 + h) * kSfaMmaD)[ch];
      *reinterpret_cast<uint4*>(&dos[h * kSfaMmaDStride + ch * 8]) = v;
    }
    // delta = dO . O per head (16 threads per head), and the forward statistics
    {
      const int ah = tid >> 4;
      float part = 0.f;
      if (h0 + ah < p.n1) {
        const T* o = (const T*)p.out + ((int64_t)row * p.n1 + h0 + ah) * kSfaMmaD;
        const T* gd = dout + (int64_t)(h0 + ah) * kSfaMmaD;
        for (int cc = tid & 15; cc < kSfaMmaD; cc += 16) part = fmaf(to_f32<T>(gd[cc]), to_f32<T>(o[cc]), part);
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

  // Slot tables are double-buffered and the keys of the next chunk that holds a key are fetched with
  // cp.async while the current chunk's d_key / d_value products (which do not read `ks`) run.
  auto fill_slots = [&](int32_t j0, int buf) -> int {
    int any = 0;
    if (tid < kSfaGradKeys) {
      const int32_t j = j0 + tid;
      const int32_t tok = j < slots ? sfa_slot_token(p.seq, p.sparse_block_size, ri, idx_row, j) : -1;
      const int64_t r = tok >= 0 ? key_row(p.seq, ri, tok) : -1;
      tok_s[buf][tid] = r >= 0 ? tok : -1;
      krow_s[buf][tid] = r;
      any = r >= 0;
    }
    return any;
  };
  // First chunk at or after j0 with a key: its slot table goes to `buf`; returns its start or `slots`.
  auto next_chunk = [&](int32_t j0, int buf) -> int32_t {
    while (j0 < slots) {
      if (__syncthreads_or(fill_slots(j0, buf))) break;
      j0 += kSfaGradKeys;
    }
    return j0;
  };
  auto gather_async = [&](int buf) {
    constexpr int cn = kSfaMmaD / 8, ct = kSfaMmaDq / 8;
    for (int i = tid; i < kSfaGradKeys * ct; i += NT) {
      const int k = i / ct, ch = i - k * ct;
      const int64_t kr_ = krow_s[buf][k];
      const T* src = kn;
      if (kr_ >= 0) src = ch < cn ? kn + kr_ * kSfaMmaD + ch * 8 : kr + kr_ * kSfaMmaDr + (ch - cn) * 8;
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&ks[k * kSfaMmaStride + ch * 8]);
      const int bytes = kr_ >= 0 ? 16 : 0;     // 0: the 16 bytes are zero-filled
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  int buf = 0;
  int32_t j0 = next_chunk(0, buf);
  if (j0 < slots) gather_async(buf);
  while (j0 < slots) {
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();

    // One 16-head x 8-key tile per warp: the first 4 MT warps compute S -> P, the others dP.
    {
      const bool is_s = warp < 4 * MT;
      const int m0 = ((warp >> 2) % MT) * 16;
      const int n0 = (warp & 3) * 8;
      const T* a_base = is_s ? qs + m0 * kSfaMmaStride : dos + m0 * kSfaMmaDStride;
      const int a_stride = is_s ? kSfaMmaStride : kSfaMmaDStride;
      const int ksteps = is_s ? kSfaMmaDq / 16 : kSfaMmaD / 16;
      float cs[4][4];     // four independent accumulation chains
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < 4; ++e) cs[u][e] = 0.f;
      // ldmatrix addresses: A = 16 heads x 16 columns per step (four 8x8 blocks: rows 0-7 / 8-15 of
      // columns k0.. and k0+8..), B = keys n0..n0+7 x 32 columns per two steps
      const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(
          a_base + ((lane & 7) + ((lane >> 3) & 1) * 8) * a_stride + (lane >> 4) * 8);
      const uint32_t b_addr =
          (uint32_t)__cvta_generic_to_shared(&ks[(n0 + (lane & 7)) * kSfaMmaStride + (lane >> 3) * 8]);
      for (int s = 0; s < ksteps; s += 4) {
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
      for (int e = 0; e < 4; ++e) {
        const int h = m0 + g + (e >> 1) * 8, k = n0 + 2 * c + (e & 1);
        const float v = (cs[0][e] + cs[1][e]) + (cs[2][e] + cs[3][e]);
        if (is_s) {
          const float l = sum_s[h];
          ps_f[h][k] = (tok_s[buf][k] >= 0 && l > 0.f) ? expf(v * p.scale - max_s[h]) / l : 0.f;
        } else {
          dp_f[h][k] = v;
        }
      }
    }
    __syncthreads();

    // dS, and both P and dS as high + low io-dtype parts in the layouts the products below read.
    // fp16 has a narrow exponent range: P (at most 1) is scaled by 2^13 and dS by a power of two that
    // brings the chunk's largest |dS| to about 2^13, so that neither part under- or overflows; the
    // products are scaled back in fp32 (dq_exp / dk_down below).
    float dk_down = 1.f, p_up = 1.f;
    {
      float pv[2], dsv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = tid + u * NT, h = i >> 5, k = i & 31;
        pv[u] = ps_f[h][k];
        dsv[u] = pv[u] * (dp_f[h][k] - delta_s[h]) * p.scale;
      }
      float up_k = 1.f, up_q = 1.f;
      if constexpr (kScaled) {
        float m = fmaxf(fabsf(dsv[0]), fabsf(dsv[1]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red_s[warp] = m;
        __syncthreads();
        m = red_s[0];
#pragma unroll
        for (int wv = 1; wv < NT / 32; ++wv) m = fmaxf(m, red_s[wv]);
        // (a chunk whose values are all zero must not pin the accumulator's scale: it keeps the
        // current one, or 2^100 before the first chunk with a non-zero value)
        int e = (m > 0.f && m < INFINITY) ? 13 - ilogbf(m) : min(dq_exp, 100);
        e = max(-100, min(100, e));
        if (e < dq_exp) {                 // the accumulator follows the smallest scale seen so far
          const float f = scalbnf(1.f, e - dq_exp);
#pragma unroll
          for (int t = 0; t < QT; ++t)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[t][x] *= f;
          dq_exp = e;
        }
        up_k = scalbnf(1.f, e);
        up_q = scalbnf(1.f, dq_exp);
        dk_down = scalbnf(1.f, -e);
        p_up = 8192.f;
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = tid + u * NT, h = i >> 5, k = i & 31;
        const float pp = pv[u] * p_up, dk_ = dsv[u] * up_k, dq_ = dsv[u] * up_q;
        const T ph = from_f32<T>(pp), kh = from_f32<T>(dk_), qh = from_f32<T>(dq_);
        pt_hi[k * PH + h] = ph;
        pt_lo[k * PH + h] = from_f32<T>(pp - to_f32<T>(ph));
        dst_hi[k * PH + h] = kh;
        dst_lo[k * PH + h] = from_f32<T>(dk_ - to_f32<T>(kh));
        ds_hi[h * kSfaMmaPk + k] = qh;
        ds_lo[h * kSfaMmaPk + k] = from_f32<T>(dq_ - to_f32<T>(qh));
      }
    }
    __syncthreads();

    // d_query (nope | rope) += dS . k : 16 heads x 8 QT columns per warp, 32 keys deep
#pragma unroll
    for (int k0 = 0; k0 < kSfaGradKeys; k0 += 16) {
      uint32_t ah[4], al[4];
      load_a_frag<T>(ah, ds_hi, kSfaMmaPk, qm0, k0);
      load_a_frag<T>(al, ds_lo, kSfaMmaPk, qm0, k0);
#pragma unroll
      for (int t = 0; t < QT; ++t) {
        uint32_t b0, b1;
        ldmatrix_b_trans<T>(b0, b1, &ks[k0 * kSfaMmaStride + qn0 + t * 8], kSfaMmaStride);
        mma_16816<T>(acc[t], ah, b0, b1);
        mma_16816<T>(acc[t], al, b0, b1);
      }
    }

    // look for the next chunk and, once every warp is done with `ks` (the barrier inside), start
    // fetching its keys
    const int32_t jn = next_chunk(j0 + kSfaGradKeys, buf ^ 1);
    if (jn < slots) gather_async(buf ^ 1);

    // d_key (nope | rope) += dS^T . q and d_value += P^T . dO, HB heads deep.  A warp takes 2 / MT
    // 16-key tiles x 8 QT columns of d_key and x 8 VT columns of d_value.
    {
      constexpr int KT = 2 / MT;             // key tiles per warp
      const int kt0 = MT == 2 ? (warp >> 3) : 0;
      const int vn0 = (warp & 7) * (VT * 8);
      uint32_t ah[KT][MT][4], al[KT][MT][4];
#pragma unroll
      for (int kt = 0; kt < KT; ++kt)
#pragma unroll
        for (int hs = 0; hs < MT; ++hs) {
          load_a_frag<T>(ah[kt][hs], dst_hi, PH, (kt0 + kt) * 16, hs * 16);
          load_a_frag<T>(al[kt][hs], dst_lo, PH, (kt0 + kt) * 16, hs * 16);
        }
      for (int t = 0; t < QT; ++t) {
        const int n0 = qn0 + t * 8;
        uint32_t b[MT][2];
#pragma unroll
        for (int hs = 0; hs < MT; ++hs) ldmatrix_b_trans<T>(b[hs][0], b[hs][1], &qs[hs * 16 * kSfaMmaStride + n0], kSfaMmaStride);
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          float cf[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int hs = 0; hs < MT; ++hs) {
            mma_16816<T>(cf, ah[kt][hs], b[hs][0], b[hs][1]);
            mma_16816<T>(cf, al[kt][hs], b[hs][0], b[hs][1]);
          }
          if constexpr (kScaled) {
#pragma unroll
            for (int x = 0; x < 4; ++x) cf[x] *= dk_down;
          }
          const int kr0 = (kt0 + kt) * 16 + g;
          red_tile(p.dk_acc, kSfaMmaDq, krow_s[buf][kr0], krow_s[buf][kr0 + 8], n0, cf);
        }
      }
#pragma unroll
      for (int kt = 0; kt < KT; ++kt)
#pragma unroll
        for (int hs = 0; hs < MT; ++hs) {
          load_a_frag<T>(ah[kt][hs], pt_hi, PH, (kt0 + kt) * 16, hs * 16);
          load_a_frag<T>(al[kt][hs], pt_lo, PH, (kt0 + kt) * 16, hs * 16);
        }
      for (int t = 0; t < VT; ++t) {
        const int n0 = vn0 + t * 8;
        uint32_t b[MT][2];
#pragma unroll
        for (int hs = 0; hs < MT; ++hs) ldmatrix_b_trans<T>(b[hs][0], b[hs][1], &dos[hs * 16 * kSfaMmaDStride + n0], kSfaMmaDStride);
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          float cf[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int hs = 0; hs < MT; ++hs) {
            mma_16816<T>(cf, ah[kt][hs], b[hs][0], b[hs][1]);
            mma_16816<T>(cf, al[kt][hs], b[hs][0], b[hs][1]);
          }
          if constexpr (kScaled) {
#pragma unroll
            for (int x = 0; x < 4; ++x) cf[x] *= (1.f / 8192.f);
          }
          const int kr0 = (kt0 + kt) * 16 + g;
          red_tile(p.dv_acc, kSfaMmaD, krow_s[buf][kr0], krow_s[buf][kr0 + 8], n0, cf);
        }
      }
    }
    j0 = jn;
    buf ^= 1;
  }

  // d_query / d_query_rope of this head chunk (zeros for inactive rows)
  const float dq_down = kScaled ? scalbnf(1.f, -dq_exp) : 1.f;
#pragma unroll
  for (int t = 0; t < QT; ++t) {
    const int col = qn0 + t * 8 + 2 * c;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int h = qm0 + g + half * 8;
      if (h0 + h >= p.n1) continue;
      const int64_t qh = (int64_t)row * p.n1 + h0 + h;
      T* dst = col < kSfaMmaD ? (T*)p.d_query + qh * kSfaMmaD + col : (T*)p.d_query_rope + qh * kSfaMmaDr + (col - kSfaMmaD);
      dst[0] = from_f32<T>(acc[t][2 * half] * dq_down);
      dst[1] = from_f32<T>(acc[t][2 * half + 1] * dq_down);
    }
  }
}

}  // namespace dsa
