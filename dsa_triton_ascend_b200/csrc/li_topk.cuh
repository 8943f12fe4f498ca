// Ordered top-k over one score row per thread block: radix select of the k-th key, exact tie
// cut by position, then a bitonic sort of the <= k survivors.  Replaces the library call of
// _stable_topk (lightning_indexer_triton.py:343-361): output order is (score descending,
// position ascending), unused slots hold index -1 / value 0 as the numpy golden does
// (lightning_indexer_numpy.py:66-67,94-105).
//
// Rank key: DSA_RANK_IO_DTYPE ranks the score rounded to the q/k dtype (16-bit key, what the
// golden ranks); DSA_RANK_FP32 ranks the raw fp32 score (what the reference device path ranks).
#pragma once

#include "li_score_simt.cuh"

namespace dsa {

constexpr int kTopkThreads = 512;
constexpr int kTopkKeyCache = 16384;  // keys of rows up to this length are cached in shared memory
constexpr int kTopkMaxCount = 8192;   // largest supported sparse_count

__device__ __forceinline__ uint32_t sortable_f32(float x) {
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Monotone unsigned key of a score: larger key == better rank.  Both zeros map to one key
// (numpy compares -0.0 == 0.0, so the golden breaks such ties by position).
template <typename T, bool kRank16>
__device__ __forceinline__ uint32_t rank_key(float x) {
  if (kRank16) {
    T r = from_f32<T>(x);
    uint16_t h = *reinterpret_cast<uint16_t*>(&r);
    if ((h & 0x7FFFu) == 0) h = 0;
    return (h & 0x8000u) ? (uint32_t)(uint16_t)(~h) : (uint32_t)(h | 0x8000u);
  }
  return sortable_f32(x + 0.f);
}

// Exclusive prefix sum over 256 bins held one per thread (threads 0..255); `warp_tot` is 8 words.
__device__ __forceinline__ uint32_t bins_exclusive_prefix(uint32_t v, uint32_t* warp_tot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (warp < 8 && lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  uint32_t base = 0;
  if (warp < 8) {
    for (int w = 0; w < warp; ++w) base += warp_tot[w];
  }
  return base + inc - v;
}

// grid = rows * n2; block = 512 threads; dynamic smem = sort_cap * 8 + kTopkKeyCache * 4 bytes.
template <typename T, bool kRank16>
__global__ void __launch_bounds__(kTopkThreads) li_topk_kernel(LiDev p, const float* __restrict__ scores,
                                                               int64_t ld, int32_t sort_cap) {
  extern __shared__ __align__(16) unsigned char topk_smem[];
  uint64_t* sbuf = reinterpret_cast<uint64_t*>(topk_smem);
  uint32_t* kcache = reinterpret_cast<uint32_t*>(sbuf + sort_cap);
  __shared__ uint32_t hist[256];
  __shared__ uint32_t warp_tot[8];
  __shared__ uint32_t sh_digit, sh_below, sh_cnt, sh_count;

  const int tid = threadIdx.x;
  const int32_t rown = blockIdx.x;
  const int32_t row = rown / p.n2;
  const RowInfo ri = row_info(p.seq, row);
  const int32_t n = ri.visible;
  const int32_t K = p.sparse_count;
  const int32_t nsel = min(n, K);
  int32_t* oi = p.out_indices + (int64_t)rown * K;
  T* ov = (p.return_value && p.out_values != nullptr) ? (T*)p.out_values + (int64_t)rown * K : nullptr;

  for (int i = nsel + tid; i < K; i += kTopkThreads) {
    oi[i] = -1;
    if (ov) ov[i] = from_f32<T>(0.f);
  }
  if (nsel == 0) return;

  const float* s = scores + (int64_t)rown * ld;
  const bool cached = n <= kTopkKeyCache;
  if (cached) {
    for (int i = tid; i < n; i += kTopkThreads) kcache[i] = rank_key<T, kRank16>(s[i]);
    __syncthreads();
  }
  auto key_at = [&](int i) -> uint32_t { return cached ? kcache[i] : rank_key<T, kRank16>(s[i]); };

  uint32_t thr_key = 0, pos_limit = 0xFFFFFFFFu;
  if (n > K) {
    // ---- radix select on the key bytes, most significant first (bins reversed: best first)
    uint32_t prefix = 0, mask = 0, remaining = (uint32_t)K, eq_count = 0;
    constexpr int kKeyBytes = kRank16 ? 2 : 4;
#pragma unroll 1
    for (int byte = kKeyBytes - 1; byte >= 0; --byte) {
      const int shift = byte * 8;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (int i = tid; i < n; i += kTopkThreads) {
        uint32_t key = key_at(i);
        if ((key & mask) == prefix) atomicAdd(&hist[255 - ((key >> shift) & 255u)], 1u);
      }
      __syncthreads();
      uint32_t cnt = tid < 256 ? hist[tid] : 0;
      uint32_t below = bins_exclusive_prefix(cnt, warp_tot);
      if (tid < 256 && below < remaining && remaining <= below + cnt) {
        sh_digit = 255 - tid; sh_below = below; sh_cnt = cnt;
      }
      __syncthreads();
      prefix |= sh_digit << shift;
      mask |= 0xFFu << shift;
      remaining -= sh_below;
      eq_count = sh_cnt;
      __syncthreads();
    }
    thr_key = prefix;
    if (remaining < eq_count) {
      // ---- more ties than slots: keep the `remaining` smallest positions (ascending radix select)
      const int pbytes = n <= 256 ? 1 : (n <= 65536 ? 2 : 3);
      uint32_t pprefix = 0, pmask = 0;
#pragma unroll 1
      for (int byte = pbytes - 1; byte >= 0; --byte) {
        const int shift = byte * 8;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int i = tid; i < n; i += kTopkThreads) {
          if (((uint32_t)i & pmask) == pprefix && key_at(i) == thr_key)
            atomicAdd(&hist[((uint32_t)i >> shift) & 255u], 1u);
        }
        __syncthreads();
        uint32_t cnt = tid < 256 ? hist[tid] : 0;
        uint32_t below = bins_exclusive_prefix(cnt, warp_tot);
        if (tid < 256 && below < remaining && remaining <= below + cnt) {
          sh_digit = tid; sh_below = below;
        }
        __syncthreads();
        pprefix |= sh_digit << shift;
        pmask |= 0xFFu << shift;
        remaining -= sh_below;
        __syncthreads();
      }
      pos_limit = pprefix;
    }
  }

  // ---- compact the survivors as (key, ~position) composites; all composites are distinct
  if (tid == 0) sh_count = 0;
  __syncthreads();
  for (int i = tid; i < n; i += kTopkThreads) {
    uint32_t key = key_at(i);
    if (key > thr_key || (key == thr_key && (uint32_t)i <= pos_limit)) {
      uint32_t slot = atomicAdd(&sh_count, 1u);
      if (slot < (uint32_t)sort_cap) sbuf[slot] = ((uint64_t)key << 32) | (uint64_t)(0xFFFFFFFFu - (uint32_t)i);
    }
  }
  int32_t p2 = 1;
  while (p2 < nsel) p2 <<= 1;
  for (int i = nsel + tid; i < p2; i += kTopkThreads) sbuf[i] = 0ull;
  __syncthreads();

  // ---- bitonic sort, descending
  for (int size = 2; size <= p2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < (p2 >> 1); t += kTopkThreads) {
        int i = 2 * t - (t & (stride - 1));
        int j = i + stride;
        uint64_t a = sbuf[i], b = sbuf[j];
        bool desc = (i & size) == 0;
        if ((a < b) == desc) { sbuf[i] = b; sbuf[j] = a; }
      }
      __syncthreads();
    }
  }

  for (int i = tid; i < nsel; i += kTopkThreads) {
    uint32_t pos = 0xFFFFFFFFu - (uint32_t)sbuf[i];
    oi[i] = (int32_t)pos;
    if (ov) ov[i] = from_f32<T>(s[pos] + 0.f);
  }
}

}  // namespace dsa
