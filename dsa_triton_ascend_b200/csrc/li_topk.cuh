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
  const uint32_t lt = (1u << (tid & 31)) - 1u;
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
  // keys of positions i..i+3 (i a multiple of 4; rows start 16-byte aligned); 0 past the end of the
  // row (real keys are >= 1)
  auto keys4_at = [&](int i, uint32_t* k4) {
    if (i + 3 < n) {
      if (cached) {
        const uint4 v = *reinterpret_cast<const uint4*>(kcache + i);
        k4[0] = v.x; k4[1] = v.y; k4[2] = v.z; k4[3] = v.w;
      } else {
        const float4 v = *reinterpret_cast<const float4*>(s + i);
        k4[0] = rank_key<T, kRank16>(v.x); k4[1] = rank_key<T, kRank16>(v.y);
        k4[2] = rank_key<T, kRank16>(v.z); k4[3] = rank_key<T, kRank16>(v.w);
      }
    } else {
#pragma unroll
      for (int u = 0; u < 4; ++u) k4[u] = i + u < n ? key_at(i + u) : 0u;
    }
  };

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
      // 2 x 4 keys per thread in flight (16-byte loads): long rows are not cached in shared memory,
      // and one 4-byte dependent load per iteration leaves the pass bound by memory latency
      for (int i0 = 0; i0 < n; i0 += 8 * kTopkThreads) {
        uint32_t key[8];
        keys4_at(i0 + 4 * tid, key);
        keys4_at(i0 + 4 * kTopkThreads + 4 * tid, key + 4);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (key[u] != 0u && (key[u] & mask) == prefix) atomicAdd(&hist[255 - ((key[u] >> shift) & 255u)], 1u);
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
        for (int i0 = 0; i0 < n; i0 += 8 * kTopkThreads) {
          uint32_t key[8];
          keys4_at(i0 + 4 * tid, key);
          keys4_at(i0 + 4 * kTopkThreads + 4 * tid, key + 4);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t i = (uint32_t)(i0 + (u >> 2) * 4 * kTopkThreads + 4 * tid + (u & 3));
            if (key[u] == thr_key && (i & pmask) == pprefix) atomicAdd(&hist[(i >> shift) & 255u], 1u);
          }
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
  for (int i0 = 0; i0 < n; i0 += 8 * kTopkThreads) {
    // 2 x 4 keys per thread in flight; one shared-memory add per warp and key slot (the order
    // inside the buffer does not matter: it is sorted below)
    uint32_t key[8];
    keys4_at(i0 + 4 * tid, key);
    keys4_at(i0 + 4 * kTopkThreads + 4 * tid, key + 4);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + (u >> 2) * 4 * kTopkThreads + 4 * tid + (u & 3);
      const bool keep = key[u] != 0u && (key[u] > thr_key || (key[u] == thr_key && (uint32_t)i <= pos_limit));
      const uint32_t km = __ballot_sync(0xffffffffu, keep);
      uint32_t base = 0;
      if ((tid & 31) == 0 && km) base = atomicAdd(&sh_count, (uint32_t)__popc(km));
      base = __shfl_sync(0xffffffffu, base, 0);
      if (keep) {
        const uint32_t slot = base + __popc(km & lt);
        if (slot < (uint32_t)sort_cap) sbuf[slot] = ((uint64_t)key[u] << 32) | (uint64_t)(0xFFFFFFFFu - (uint32_t)i);
      }
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

// ------------------------------------------------------------------------------------------------
// Fast path for rows of up to 8192 visible keys and sparse_count <= 512 * E (E = 1, 2, 4):
//   * every thread keeps 16 rank keys in registers (position = j * 512 + tid);
//   * the k-th key is found by bisection on the key value: each step counts the keys >= mid with a
//     warp reduction and one shared-memory add per warp (no histogram, hence no atomic contention
//     on the few exponent bins that hold nearly all scores);
//   * ties at the threshold are cut by a second bisection on the position;
//   * the survivors are written as composites (key, ~position) and sorted by a bitonic network
//     that runs in registers / warp shuffles, touching shared memory only for the four largest
//     strides;
//   * values are rebuilt from the composite, so the scores are read exactly once.
// Composite: 32 bits (16-bit key | 16-bit ~position) when ranking the io dtype, else 64 bits.
// ------------------------------------------------------------------------------------------------
constexpr int kTopkFastKeys = 16;   // keys per thread -> rows of up to 8192 visible keys

template <bool kRank16> struct TopkComposite { typedef uint64_t type; };
template <> struct TopkComposite<true> { typedef uint32_t type; };

template <typename C> __device__ __forceinline__ C shfl_xor_c(C v, int m);
template <> __device__ __forceinline__ uint32_t shfl_xor_c<uint32_t>(uint32_t v, int m) {
  return __shfl_xor_sync(0xffffffffu, v, m);
}
template <> __device__ __forceinline__ uint64_t shfl_xor_c<uint64_t>(uint64_t v, int m) {
  return __shfl_xor_sync(0xffffffffu, (unsigned long long)v, m);
}

// Block-wide sum of one small integer per thread; `slot` must be a zeroed shared counter that is
// not reused before the next __syncthreads of the caller's own loop.
__device__ __forceinline__ uint32_t block_count(uint32_t c, uint32_t* slot) {
  const uint32_t w = __reduce_add_sync(0xffffffffu, c);
  if ((threadIdx.x & 31) == 0 && w) atomicAdd(slot, w);
  __syncthreads();
  return *slot;
}

template <typename T, bool kRank16, int E>
__global__ void __launch_bounds__(kTopkThreads) li_topk_fast_kernel(LiDev p, const float* __restrict__ scores,
                                                                    int64_t ld) {
  typedef typename TopkComposite<kRank16>::type C;
  constexpr int P2 = kTopkThreads * E;
  __shared__ C sbuf[P2];
  __shared__ uint32_t counters[64];
  __shared__ uint32_t sh_count;

  const int tid = threadIdx.x;
  const int32_t rown = blockIdx.x;
  const int32_t row = rown / p.n2;
  const RowInfo ri = row_info(p.seq, row);
  const int32_t n = ri.visible;
  const int32_t K = p.sparse_count;
  const int32_t nsel = min(n, K);
  int32_t* oi = p.out_indices + (int64_t)rown * K;
  T* ov = (p.return_value && p.out_values != nullptr) ? (T*)p.out_values + (int64_t)rown * K : nullptr;

  if (nsel == 0) {
    for (int i = tid; i < K; i += kTopkThreads) {
      oi[i] = -1;
      if (ov) ov[i] = from_f32<T>(0.f);
    }
    return;
  }
  const float* s = scores + (int64_t)rown * ld;
  uint32_t key[kTopkFastKeys];
#pragma unroll
  for (int j = 0; j < kTopkFastKeys; ++j) {
    const int pos = j * kTopkThreads + tid;
    key[j] = pos < n ? rank_key<T, kRank16>(s[pos]) : 0u;   // 0 is below every real key
  }
  if (tid < 64) counters[tid] = 0;
  if (tid == 0) sh_count = 0;
  __syncthreads();

  uint32_t thr_key = 0, pos_limit = 0xFFFFFFFFu;
  if (n > K) {
    // largest T with count(key >= T) >= K
    uint32_t lo = 1, hi = kRank16 ? 0xFFFFu : 0xFFFFFFFFu;
    constexpr int kSteps = kRank16 ? 16 : 32;
    int slot = 0;
#pragma unroll 1
    for (int it = 0; it < kSteps; ++it, ++slot) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + ((hi - lo) & 1u);   // upper middle
      uint32_t c = 0;
#pragma unroll
      for (int j = 0; j < kTopkFastKeys; ++j) c += key[j] >= mid;
      const uint32_t total = block_count(c, &counters[slot]);
      if (total >= (uint32_t)K) lo = mid; else hi = mid - 1;
      if (lo == hi) { ++slot; break; }
    }
    thr_key = lo;
    uint32_t cgt = 0, ceq = 0;
#pragma unroll
    for (int j = 0; j < kTopkFastKeys; ++j) { cgt += key[j] > thr_key; ceq += key[j] == thr_key; }
    const uint32_t n_gt = block_count(cgt, &counters[slot++]);
    const uint32_t n_eq = block_count(ceq, &counters[slot++]);
    const uint32_t need = (uint32_t)K - n_gt;
    if (need < n_eq) {
      // smallest P with count(key == T and pos <= P) >= need
      uint32_t plo = 0, phi = (uint32_t)n - 1;
#pragma unroll 1
      while (plo < phi) {
        const uint32_t mid = plo + ((phi - plo) >> 1);
        uint32_t c = 0;
#pragma unroll
        for (int j = 0; j < kTopkFastKeys; ++j)
          c += (key[j] == thr_key) && ((uint32_t)(j * kTopkThreads + tid) <= mid);
        const uint32_t total = block_count(c, &counters[slot++]);
        if (total >= need) phi = mid; else plo = mid + 1;
      }
      pos_limit = plo;
    }
  }

  // ---- survivors -> composites in shared memory (any order: the sort fixes it)
#pragma unroll
  for (int j = 0; j < kTopkFastKeys; ++j) {
    const uint32_t pos = j * kTopkThreads + tid;
    const bool sel = (int32_t)pos < n && (key[j] > thr_key || (key[j] == thr_key && pos <= pos_limit));
    const uint32_t m = __ballot_sync(0xffffffffu, sel);
    uint32_t base = 0;
    if ((tid & 31) == 0 && m) base = atomicAdd(&sh_count, __popc(m));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (sel) {
      const uint32_t slot = base + __popc(m & ((1u << (tid & 31)) - 1u));
      if (slot < (uint32_t)P2) {
        if (kRank16) sbuf[slot] = (C)((key[j] << 16) | (0xFFFFu - pos));
        else sbuf[slot] = (C)(((uint64_t)key[j] << 32) | (uint64_t)(0xFFFFFFFFu - pos));
      }
    }
  }
  __syncthreads();

  // ---- bitonic sort, descending; element e = tid * E + j
  C v[E];
#pragma unroll
  for (int j = 0; j < E; ++j) {
    const int e = tid * E + j;
    v[j] = e < nsel ? sbuf[e] : (C)0;
  }
#pragma unroll 1
  for (int size = 2; size <= P2; size <<= 1) {
#pragma unroll 1
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (stride >= 32 * E) {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < E; ++j) sbuf[tid * E + j] = v[j];
        __syncthreads();
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const int e = tid * E + j;
          const C o = sbuf[e ^ stride];
          const bool take_max = (((e & stride) == 0) == ((e & size) == 0));
          v[j] = take_max ? (v[j] > o ? v[j] : o) : (v[j] < o ? v[j] : o);
        }
      } else if (stride >= E) {
        const int m = stride / E;
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const int e = tid * E + j;
          const C o = shfl_xor_c<C>(v[j], m);
          const bool take_max = (((e & stride) == 0) == ((e & size) == 0));
          v[j] = take_max ? (v[j] > o ? v[j] : o) : (v[j] < o ? v[j] : o);
        }
      } else {
        // partner inside the thread: compile-time strides keep v[] in registers
#pragma unroll
        for (int S = E / 2; S > 0; S >>= 1) {
          if (stride == S) {
#pragma unroll
            for (int j = 0; j < E; ++j) {
              if ((j & S) == 0) {
                const int e = tid * E + j;
                const bool desc = (e & size) == 0;
                const C a = v[j], b = v[j | S];
                const bool sw = desc ? (a < b) : (a > b);
                v[j] = sw ? b : a;
                v[j | S] = sw ? a : b;
              }
            }
          }
        }
      }
    }
  }

  // ---- emit: positions and values come out of the composites
#pragma unroll
  for (int j = 0; j < E; ++j) {
    const int e = tid * E + j;
    if (e < K) {
      if (e < nsel) {
        uint32_t pos, k32;
        if (kRank16) { pos = 0xFFFFu - ((uint32_t)v[j] & 0xFFFFu); k32 = (uint32_t)v[j] >> 16; }
        else { pos = 0xFFFFFFFFu - (uint32_t)v[j]; k32 = (uint32_t)((uint64_t)v[j] >> 32); }
        oi[e] = (int32_t)pos;
        if (ov) {
          if (kRank16) {
            const uint16_t h = (k32 & 0x8000u) ? (uint16_t)(k32 & 0x7FFFu) : (uint16_t)(~k32);
            ov[e] = *reinterpret_cast<const T*>(&h);
          } else {
            const uint32_t u = (k32 & 0x80000000u) ? (k32 & 0x7FFFFFFFu) : ~k32;
            ov[e] = from_f32<T>(__uint_as_float(u));
          }
        }
      } else {
        oi[e] = -1;
        if (ov) ov[e] = from_f32<T>(0.f);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Radix path (io-dtype ranking, rows of up to 8192 visible keys, sparse_count <= 2048).
// The rank key has only 16 bits, so the whole job is done with counting instead of comparing:
//   1. threshold: two 256-bin histograms (high byte, then low byte inside the chosen bin), filled
//      with warp-aggregated adds (__match_any_sync) because nearly all scores share a few bins;
//   2. ordered compaction: per (round, warp) counts of "key > T" and "key == T" elements are
//      prefix-summed in position order, which both places the survivors in ascending position
//      and cuts the ties at the threshold to the first `need` positions without any search;
//   3. stable LSD radix sort of the <= 2048 survivors on the key, kSortBits bits per pass, descending;
//      passes over bit groups in which all survivors agree are skipped (usually 1-2 of the 4).
//      Equal keys keep their ascending position order, which is the required tie-break.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_tot /*[16]*/, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  uint32_t base = 0, all = 0;
#pragma unroll
  for (int w = 0; w < kTopkThreads / 32; ++w) {
    const uint32_t t = warp_tot[w];
    if (w < warp) base += t;
    all += t;
  }
  if (total) *total = all;
  __syncthreads();   // warp_tot may be reused right away
  return base + inc - v;
}

// Mask of the lanes whose kBits-bit digit equals this lane's (one ballot per bit; cheaper than a match).
template <int kBits>
__device__ __forceinline__ uint32_t same_digit(uint32_t d) {
  uint32_t m = 0xffffffffu;
#pragma unroll
  for (int b = 0; b < kBits; ++b) {
    const uint32_t v = __ballot_sync(0xffffffffu, (d >> b) & 1u);
    m &= ((d >> b) & 1u) ? v : ~v;
  }
  return m;
}
constexpr int kSortBits = 4;                       // digit width of the survivor sort
constexpr int kSortBins = 1 << kSortBits;
constexpr int kSortPasses = (16 + kSortBits - 1) / kSortBits;

template <typename T, int E>
__global__ void __launch_bounds__(kTopkThreads, 2) li_topk_radix_kernel(LiDev p, const float* __restrict__ scores,
                                                                     int64_t ld) {
  constexpr int P2 = kTopkThreads * E;
  constexpr int NW = kTopkThreads / 32;
  __shared__ uint32_t buf[2][P2];
  constexpr int TN = kSortBins * E * NW;          // (digit, round, warp) counters of a sort pass
  __shared__ uint32_t tab[TN < 512 ? 512 : TN];   // also holds the 2 x 256 compaction counters
  __shared__ uint32_t hist[256];
  __shared__ uint32_t warp_tot[NW];
  __shared__ uint32_t sh_a, sh_b, sh_c, sh_diff, sh_ref;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  const int32_t rown = blockIdx.x;
  const int32_t row = rown / p.n2;
  const RowInfo ri = row_info(p.seq, row);
  const int32_t n = ri.visible;
  const int32_t K = p.sparse_count;
  const int32_t nsel = min(n, K);
  int32_t* oi = p.out_indices + (int64_t)rown * K;
  T* ov = (p.return_value && p.out_values != nullptr) ? (T*)p.out_values + (int64_t)rown * K : nullptr;
  if (nsel == 0) {
    for (int i = tid; i < K; i += kTopkThreads) {
      oi[i] = -1;
      if (ov) ov[i] = from_f32<T>(0.f);
    }
    return;
  }
  const float* s = scores + (int64_t)rown * ld;
  // rounds (of 512 positions) that hold visible keys; the per-key loops below skip the rest
  const int rounds = (n + kTopkThreads - 1) / kTopkThreads;
  uint32_t key[kTopkFastKeys];
#pragma unroll
  for (int j = 0; j < kTopkFastKeys; ++j) {
    const int pos = j * kTopkThreads + tid;
    key[j] = (j < rounds && pos < n) ? rank_key<T, true>(s[pos]) : 0u;   // real keys are >= 1
  }

  // ---- 1. threshold key T, number of keys above it and of ties to keep
  uint32_t thr = 0, need = 0;
  if (n > K) {
    uint32_t remaining = (uint32_t)K, hi = 0;
#pragma unroll 1
    for (int level = 0; level < 2; ++level) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
#pragma unroll
      for (int j = 0; j < kTopkFastKeys; ++j) {
        if (j >= rounds) break;
        const bool in = key[j] != 0 && (level == 0 || (key[j] >> 8) == hi);
        const uint32_t d = level == 0 ? (key[j] >> 8) : (key[j] & 255u);
        if (level == 0) {
          // high byte: nearly all keys share a few values, so add once per group of equal values
          const uint32_t vm = __ballot_sync(0xffffffffu, in);
          const uint32_t m = __match_any_sync(0xffffffffu, d) & vm;
          if (in && (m & lt) == 0) atomicAdd(&hist[255 - d], __popc(m));
        } else if (in) {
          atomicAdd(&hist[255 - d], 1u);   // low byte inside the chosen bin: spread over the bins
        }
      }
      __syncthreads();
      const uint32_t cnt = tid < 256 ? hist[tid] : 0;
      const uint32_t below = block_exclusive_scan(cnt, warp_tot, nullptr);
      if (tid < 256 && below < remaining && remaining <= below + cnt) { sh_a = 255 - tid; sh_b = below; }
      __syncthreads();
      if (level == 0) hi = sh_a; else thr = (hi << 8) | sh_a;
      remaining -= sh_b;
      __syncthreads();
    }
    need = remaining;   // ties at the threshold that still fit
  } else {
    thr = 0;            // every real key is above 0: everything is kept
  }

  // ---- 2. ordered compaction through per (round, warp) counters
  uint32_t* cnt_g = tab;          // [16 rounds][16 warps]
  uint32_t* cnt_e = tab + 256;
#pragma unroll
  for (int j = 0; j < kTopkFastKeys; ++j) {
    uint32_t g = 0, e = 0;
    if (j < rounds) {
      g = __ballot_sync(0xffffffffu, key[j] > thr);
      e = __ballot_sync(0xffffffffu, thr != 0 && key[j] == thr);
    }
    if (lane == 0) { cnt_g[j * NW + warp] = __popc(g); cnt_e[j * NW + warp] = __popc(e); }
  }
  __syncthreads();
  {
    // threads 0..255 scan the "above" counters, 256..511 the "tie" counters (both in position order)
    const uint32_t v = tab[tid];
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    uint32_t base = 0;
    const int w0 = warp < 8 ? 0 : 8;
    for (int w = w0; w < warp; ++w) base += warp_tot[w];
    if (tid == 0) {
      uint32_t g = 0;
      for (int w = 0; w < 8; ++w) g += warp_tot[w];
      sh_c = g;   // number of keys above the threshold
      sh_diff = 0;
      sh_ref = thr ? thr : key[0];   // some key that is kept (position 0 is always visible)
    }
    __syncthreads();
    tab[tid] = base + inc - v;
  }
  __syncthreads();
  const uint32_t n_gt = sh_c, ref = sh_ref;
  uint32_t diff = 0;   // bits in which some kept key differs from `ref`
#pragma unroll
  for (int j = 0; j < kTopkFastKeys; ++j) {
    if (j >= rounds) break;
    const uint32_t pos = j * kTopkThreads + tid;
    const uint32_t entry = (key[j] << 16) | pos;
    const bool is_g = key[j] > thr, is_e = thr != 0 && key[j] == thr;
    const uint32_t g = __ballot_sync(0xffffffffu, is_g);
    const uint32_t e = __ballot_sync(0xffffffffu, is_e);
    if (is_g) {
      buf[0][cnt_g[j * NW + warp] + __popc(g & lt)] = entry;
      diff |= key[j] ^ ref;
    } else if (is_e) {
      const uint32_t ord = cnt_e[j * NW + warp] + __popc(e & lt);
      if (ord < need) buf[0][n_gt + ord] = entry;
    }
  }
  diff = __reduce_or_sync(0xffffffffu, diff);
  if (lane == 0 && diff) atomicOr(&sh_diff, diff);
  for (int i = nsel + tid; i < P2; i += kTopkThreads) buf[0][i] = 0x0000FFFFu;   // padding: key 0 sorts last
  __syncthreads();
  const uint32_t differing = sh_diff & 0xFFFFu;

  // ---- 3. stable LSD radix sort on the key, descending (digit' = bins - 1 - digit); digits of
  // kSortBits = 4 bits: measured 0.475 ms on 8192 x 8192, k = 2048 against 0.51 (5 bits) and 0.60 (6 bits)
  int cur = 0;
#pragma unroll 1
  for (int g = 0; g < kSortPasses; ++g) {
    if (((differing >> (kSortBits * g)) & (kSortBins - 1u)) == 0) continue;
    for (int i = tid; i < TN; i += kTopkThreads) tab[i] = 0;
    __syncthreads();
    uint32_t ent[E], rk[E], dg[E];
#pragma unroll
    for (int r = 0; r < E; ++r) {
      ent[r] = buf[cur][r * kTopkThreads + tid];
      dg[r] = (kSortBins - 1u) - ((ent[r] >> (16 + kSortBits * g)) & (kSortBins - 1u));
      const uint32_t m = same_digit<kSortBits>(dg[r]);
      rk[r] = __popc(m & lt);
      if (rk[r] == 0) tab[(dg[r] * E + r) * NW + warp] = __popc(m);
    }
    __syncthreads();
    {
      // exclusive scan of the (digit, round, warp) counters
      constexpr int PER = (TN + kTopkThreads - 1) / kTopkThreads;
      uint32_t loc[PER], sum = 0;
#pragma unroll
      for (int q = 0; q < PER; ++q) {
        loc[q] = tid * PER + q < TN ? tab[tid * PER + q] : 0u;
        sum += loc[q];
      }
      uint32_t base = block_exclusive_scan(sum, warp_tot, nullptr);
#pragma unroll
      for (int q = 0; q < PER; ++q) {
        if (tid * PER + q < TN) tab[tid * PER + q] = base;
        base += loc[q];
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < E; ++r) buf[cur ^ 1][tab[(dg[r] * E + r) * NW + warp] + rk[r]] = ent[r];
    __syncthreads();
    cur ^= 1;
  }

  // ---- 4. emit
  for (int i = tid; i < K; i += kTopkThreads) {
    if (i < nsel) {
      const uint32_t e = buf[cur][i];
      oi[i] = (int32_t)(e & 0xFFFFu);
      if (ov) {
        const uint32_t k16 = e >> 16;
        const uint16_t h = (k16 & 0x8000u) ? (uint16_t)(k16 & 0x7FFFu) : (uint16_t)(~k16);
        ov[i] = *reinterpret_cast<const T*>(&h);
      }
    } else {
      oi[i] = -1;
      if (ov) ov[i] = from_f32<T>(0.f);
    }
  }
}

}  // namespace dsa
