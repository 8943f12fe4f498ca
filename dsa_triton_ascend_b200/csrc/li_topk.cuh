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

#include <type_traits>

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
// Bin path (io-dtype ranking, rows of up to 8192 visible keys, sparse_count <= 2048): selection and
// ordering from ONE histogram of the row on a linear scale of the score.
//
// Every key gets a bin b = floor((hi - x) / width), 4096 bins over [mean - 3 s, mean + 5 s] of the
// row (s = 1.25 x the mean absolute deviation, which a few outliers barely move; values outside are
// clamped to the end bins).  The bin is monotone in the score, so with bin 0 the best:
//   * the exclusive prefix sum of the bin counts is, for every bin, the output slot at which its
//     members start, and the bin in which the prefix crosses sparse_count holds the threshold;
//   * members of the bins before that one all survive; of the crossing bin the `need` best survive,
//     found by ranking its few members against each other (bisection on the composite when the bin
//     is large);
//   * survivors are dropped into their bin's slot range in arrival order (one shared-memory add),
//     and each then finds its final slot by counting the members of its own bin that precede it in
//     (key descending, position ascending) order.  Bins hold a handful of members (2048 survivors
//     over ~2000 bins), so this costs a few compares per survivor instead of the 2-4 counting
//     passes over all survivors of a radix sort.
// Rows whose scores pile into few bins (all equal, or a scale dominated by outliers) stay correct:
// bins of more than kBinSmall members are ordered by whole warps, members x members.
// Four CTAs per SM (32 registers, a few spilled words): measured faster than three or two - the
// phases are short dependent chains separated by block barriers, and more resident CTAs hide them.
// ------------------------------------------------------------------------------------------------
// Development aid, compiled only with -DDSA_TOPK_PROFILE: cycles per phase of one CTA (the row at
// three quarters of the grid), read back with dsa_debug_topk_profile().
#ifdef DSA_TOPK_PROFILE
__device__ long long g_topk_prof[16];
#define TOPK_PROF_DECL long long tp_t = clock64(); int tp_i = 0
#define TOPK_PROF() do { if (threadIdx.x == 0 && blockIdx.x == (gridDim.x / 4) * 3) { \
    const long long tp_n = clock64(); g_topk_prof[tp_i] = tp_n - tp_t; tp_t = tp_n; } ++tp_i; } while (0)
#else
#define TOPK_PROF_DECL
#define TOPK_PROF()
#endif

constexpr int kBinCount = 4096;
constexpr int kBinSmall = 16;    // bins up to this size are ordered by their own members
constexpr int kBinSide = 128;    // crossing bins up to this size are cut by ranking, larger ones by bisection
constexpr int kBinBigList = 128; // a row has at most 2048 / 17 = 120 bins above kBinSmall

template <typename T>
__device__ __forceinline__ T key16_bits(uint32_t k16) {
  const uint16_t h = (k16 & 0x8000u) ? (uint16_t)(k16 & 0x7FFFu) : (uint16_t)(~k16);
  return *reinterpret_cast<const T*>(&h);
}

__device__ __forceinline__ int32_t score_bin(float x, float hi, float inv_w) {
  return min(max(__float2int_rd((hi - x) * inv_w), 0), kBinCount - 1);
}

// Sums of two floats per thread, returned to every thread (same summation order everywhere).
__device__ __forceinline__ float2 block_sum2_f32(float u, float v, float2* part /*[16]*/) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    u += __shfl_xor_sync(0xffffffffu, u, o);
    v += __shfl_xor_sync(0xffffffffu, v, o);
  }
  if (lane == 0) part[threadIdx.x >> 5] = make_float2(u, v);
  __syncthreads();
  float2 t = part[lane & (kTopkThreads / 32 - 1)];
#pragma unroll
  for (int o = kTopkThreads / 64; o > 0; o >>= 1) {
    t.x += __shfl_xor_sync(0xffffffffu, t.x, o);
    t.y += __shfl_xor_sync(0xffffffffu, t.y, o);
  }
  return t;
}

// Rank key of a score already rounded to the io dtype (same order as rank_key<T, true>).
template <typename T>
__device__ __forceinline__ uint32_t rank_key_of(T r) {
  uint16_t h = *reinterpret_cast<uint16_t*>(&r);
  if ((h & 0x7FFFu) == 0) h = 0;
  return (h & 0x8000u) ? (uint32_t)(uint16_t)(~h) : (uint32_t)(h | 0x8000u);
}

template <typename T, int E>
__global__ void __launch_bounds__(kTopkThreads, 4) li_topk_bins_kernel(LiDev p, const float* __restrict__ scores,
                                                                    int64_t ld) {
  constexpr int P2 = kTopkThreads * E;
  constexpr int NW = kTopkThreads / 32;
  __shared__ __align__(16) uint32_t hist[kBinCount];   // counts, then slot cursors
  __shared__ uint32_t buf[P2];                         // survivors by bin, any order inside a bin
  __shared__ uint16_t bbin[P2];                        // their bins
  __shared__ uint32_t outs[P2];                        // survivors in output order
  __shared__ uint32_t side[kBinSide];                  // members of the crossing bin
  __shared__ uint32_t biglist[kBinBigList];
  __shared__ float2 part[NW];
  __shared__ uint32_t warp_tot[NW];
  __shared__ uint32_t counters[40];
  __shared__ uint32_t sh_bstar, sh_need, sh_cstar, sh_base, sh_side, sh_big;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
  // groups of 4 * 512 positions that hold visible keys: the per-key loops below leave at the first
  // group without one (a branch every thread of the block takes alike - predicated-off instructions
  // of an unrolled loop still take issue slots, which is what this kernel is short of)
  const int groups = (n + 4 * kTopkThreads - 1) / (4 * kTopkThreads);
  TOPK_PROF_DECL;

  // ---- 1. scale of the row from a sample of up to 512 scores spread over it: centre = their mean,
  // spread = mean distance of a sample from its neighbouring sample (for normal scores 1.13 sigma;
  // a few outliers barely move it)
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist);
    h4[2 * tid] = make_uint4(0, 0, 0, 0);
    h4[2 * tid + 1] = make_uint4(0, 0, 0, 0);
  }
  if (tid < 40) counters[tid] = 0;
  if (tid == 0) { sh_bstar = kBinCount; sh_need = 0; sh_cstar = 0; sh_base = 0; sh_side = 0; sh_big = 0; }
  float hi, inv_w;
  {
    const int ns = min(n, kTopkThreads);
    const bool in = tid < ns;
    const int sp = n > kTopkThreads ? (int)(((int64_t)tid * n) >> 9) : tid;
    const float x = in ? round_io<T>(s[sp]) : 0.f;
    const float other = __shfl_xor_sync(0xffffffffu, x, 1);
    const float dv = (in && (tid ^ 1) < ns) ? fabsf(x - other) : 0.f;
    const float2 tot = block_sum2_f32(x, dv, part);
    const float mean = tot.x / (float)ns;
    const float sdev = 0.9f * (tot.y / (float)ns);
    hi = mean + 5.f * sdev;
    inv_w = sdev > 0.f ? (float)kBinCount / (8.f * sdev) : 0.f;
    if (!(fabsf(hi) <= 3.0e38f) || !(inv_w <= 3.0e38f)) { hi = 0.f; inv_w = 0.f; }   // infinities / NaN in the sample
  }
  TOPK_PROF();   // 0: scale

  // ---- 2. load, bin, count.  Thread t holds positions 4 * (g * 512 + t) .. + 3 for g = 0..3
  // (16-byte loads; rows start 16-byte aligned and are padded to a multiple of 4 scores).
  // The io dtype is coarser than the bins wherever scores are large, so equal keys (ties, ordered by
  // position) would pile into one bin with empty bins behind it.  The next lower value of the dtype
  // lies 2^(e - mantissa bits) below a score of exponent e (half that below a positive power of
  // two); where that distance is two bins or more, the key moves down the scale by up to 63/64 of it
  // in proportion to its position.  Keys never reach a lower key's bin offset, equal keys stay in
  // position order: the bin is still monotone in (key descending, position ascending).
  constexpr int kMantBits = std::is_same<T, __half>::value ? 10 : 7;
  const float gap_scale = inv_w * (1.f / (float)(1 << kMantBits));
  const float tid4 = (float)(4 * tid);
  uint32_t key[kTopkFastKeys];   // key16 | bin << 16; bin 0xFFFF = no key at this position
#pragma unroll
  for (int g = 0; g < kTopkFastKeys; ++g) key[g] = 0xFFFF0000u;   // no key: a bin past every real one
#pragma unroll
  for (int g = 0; g < kTopkFastKeys / 4; ++g) {
    if (g >= groups) break;
    const int pos0 = 4 * (g * kTopkThreads + tid);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (pos0 < n) v = *reinterpret_cast<const float4*>(s + pos0);
    const float xs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (pos0 + u < n) {
        const T r = from_f32<T>(xs[u]);
        const float x = to_f32<T>(r);
        // equal keys are spread over the bins up to the next lower key in position order
        const uint32_t xb = __float_as_uint(x);
        const float gap = __uint_as_float(xb & 0x7F800000u) * (((xb & 0x807FFFFFu) == 0u) ? 0.5f * gap_scale : gap_scale);
        const float off = gap >= 2.f ? gap * ((tid4 + (float)(4 * g * kTopkThreads + u)) * (63.f / (64.f * 8192.f))) : 0.f;
        const int32_t b = min(max(__float2int_rd((hi - x) * inv_w + off), 0), kBinCount - 1);
        atomicAdd(&hist[b], 1u);
        key[4 * g + u] = rank_key_of<T>(r) | ((uint32_t)b << 16);
      }
    }
  }
  __syncthreads();
  TOPK_PROF();   // 1: load + histogram

  // ---- 2. slot at which every bin starts; the bin in which the count crosses K
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist);
    uint4 a = h4[2 * tid], c = h4[2 * tid + 1];
    uint32_t cnt[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
    uint32_t sum = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) sum += cnt[q];
    uint32_t inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    uint32_t run = inc - sum;
    {
      // exclusive prefix of the 16 warp totals, by shuffles inside every warp
      const uint32_t wt = warp_tot[lane & (NW - 1)];
      uint32_t winc = wt;
#pragma unroll
      for (int o = 1; o < NW; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
        if ((lane & (NW - 1)) >= o) winc += t;
      }
      run += __shfl_sync(0xffffffffu, winc - wt, warp);
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint32_t c0 = cnt[q];
      if (run < (uint32_t)K && (uint32_t)K <= run + c0) {   // the K-th best key lies in this bin
        sh_bstar = 8 * tid + q; sh_base = run; sh_need = (uint32_t)K - run; sh_cstar = c0;
      }
      cnt[q] = run;
      run += c0;
    }
    h4[2 * tid] = make_uint4(cnt[0], cnt[1], cnt[2], cnt[3]);
    h4[2 * tid + 1] = make_uint4(cnt[4], cnt[5], cnt[6], cnt[7]);
  }
  __syncthreads();
  // bins before `bstar` survive whole, bins after it not at all (no crossing: fewer than K keys);
  // of the crossing bin the `need` best survive
  const uint32_t bstar = sh_bstar, need = sh_need, cstar = sh_cstar, base_star = sh_base;
  const bool side_cut = cstar <= (uint32_t)kBinSide;
  TOPK_PROF();   // 2: scan

  // ---- 3. a large crossing bin is cut by bisection: largest C with count(members >= C) >= need.
  // (A small one goes to `side` below and is ranked there.)
  uint32_t cut = 0u;
  if (bstar < (uint32_t)kBinCount && !side_cut) {
    uint32_t lo = 1u, hi_c = 0xFFFFFFFFu;
    int slot = 0;
#pragma unroll 1
    for (int it = 0; it < 32 && lo < hi_c; ++it, ++slot) {
      const uint32_t mid = lo + ((hi_c - lo) >> 1) + ((hi_c - lo) & 1u);
      uint32_t c = 0;
#pragma unroll
      for (int j = 0; j < kTopkFastKeys; ++j) {
        const uint32_t pos = 4 * ((j >> 2) * kTopkThreads + tid) + (j & 3);
        const uint32_t comp = (key[j] << 16) | (0xFFFFu - pos);
        c += (key[j] >> 16) == bstar && comp >= mid;
      }
      const uint32_t total = block_count(c, &counters[slot]);
      if (total >= need) lo = mid; else hi_c = mid - 1u;
    }
    cut = lo;
  }

  // ---- 4. survivors into their bin's slot range (arrival order inside a bin)
#pragma unroll
  for (int j = 0; j < kTopkFastKeys; ++j) {
    if ((j >> 2) >= groups) break;
    const uint32_t b = key[j] >> 16;
    const uint32_t pos = 4 * ((j >> 2) * kTopkThreads + tid) + (j & 3);
    const uint32_t comp = (key[j] << 16) | (0xFFFFu - pos);
    if (b <= bstar) {
      if (b < bstar || (!side_cut && comp >= cut)) {
        const uint32_t slot = atomicAdd(&hist[b], 1u);
        buf[slot] = comp;
        bbin[slot] = (uint16_t)b;
      } else if (side_cut) {
        side[atomicAdd(&sh_side, 1u)] = comp;
      }
    }
  }
  __syncthreads();
  TOPK_PROF();   // 3: scatter

  // ---- 5. order inside each bin: final slot = bin start + members that precede this one
  {
    uint32_t mine[E], st[E], cn[E];
#pragma unroll
    for (int r = 0; r < E; ++r) {
      const int e = r * kTopkThreads + tid;
      mine[r] = 0u; st[r] = 0u; cn[r] = 0u;
      if (e < nsel && (!side_cut || (uint32_t)e < base_star || bstar == (uint32_t)kBinCount)) {
        mine[r] = buf[e];
        const int32_t b = bbin[e];
        st[r] = b ? hist[b - 1] : 0u;
        cn[r] = min(hist[b], (uint32_t)nsel) - st[r];
        if (cn[r] > (uint32_t)kBinSmall) {
          if ((uint32_t)e == st[r]) {
            const uint32_t i = atomicAdd(&sh_big, 1u);
            if (i < (uint32_t)kBinBigList) biglist[i] = (uint32_t)b;
          }
          cn[r] = 0u;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < E; ++r) {
      if (cn[r] != 0u) {
        uint32_t rank = 0;
        for (uint32_t q = st[r]; q < st[r] + cn[r]; ++q) rank += buf[q] > mine[r];
        outs[st[r] + rank] = mine[r];
      }
    }
    // the crossing bin: its members rank each other; the first `need` fill the last slots
    if (side_cut && (uint32_t)tid < cstar) {
      const uint32_t m = side[tid];
      uint32_t rank = 0;
      for (uint32_t q = 0; q < cstar; ++q) rank += side[q] > m;
      if (rank < need) outs[base_star + rank] = m;
    }
  }
  __syncthreads();
  TOPK_PROF();   // 4: order inside small bins
  {
    const uint32_t nbig = min(sh_big, (uint32_t)kBinBigList);
    for (uint32_t i = 0; i < nbig; ++i) {
      const uint32_t b = biglist[i];
      const uint32_t st = b ? hist[b - 1] : 0u;
      const uint32_t en = min(hist[b], (uint32_t)nsel);
      const uint32_t c = en - st;
      const bool shared_bin = c > 256u;                  // a large bin is split over all warps
      if (!shared_bin && (i % NW) != (uint32_t)warp) continue;
      for (uint32_t m0 = st + (shared_bin ? 32u * warp : 0u); m0 < en; m0 += shared_bin ? 32u * NW : 32u) {
        const uint32_t m = m0 + lane;
        const uint32_t mine = m < en ? buf[m] : 0u;
        uint32_t rank = 0;
        for (uint32_t q = st; q < en; ++q) rank += buf[q] > mine;
        if (m < en) outs[st + rank] = mine;
      }
    }
    if (nbig) __syncthreads();
  }
  TOPK_PROF();   // 5: large bins

  // ---- 6. emit: positions and values come out of the composites
  for (int i = tid; i < K; i += kTopkThreads) {
    if (i < nsel) {
      const uint32_t e = outs[i];
      oi[i] = (int32_t)(0xFFFFu - (e & 0xFFFFu));
      if (ov) ov[i] = key16_bits<T>(e >> 16);
    } else {
      oi[i] = -1;
      if (ov) ov[i] = from_f32<T>(0.f);
    }
  }
  TOPK_PROF();   // 6: emit
}

// ------------------------------------------------------------------------------------------------
// The same selection for rows of any length (io-dtype ranking, sparse_count <= 2048): the keys do
// not fit into registers, so the row is streamed twice from the score scratch (L2-resident at
// decode sizes) - once to fill the histogram, once to drop the survivors into their bins - and a
// composite is 64 bits (16-bit key | 32-bit ~position).  Everything else is li_topk_bins_kernel.
// ------------------------------------------------------------------------------------------------
template <typename T>
struct BinScale {
  float hiw, inv_w, gap_scale, pos_scale;
  // bin of the score rounded to the io dtype, at position pos (monotone in (key desc, position asc))
  __device__ __forceinline__ int32_t bin(T r, uint32_t pos) const {
    const float x = to_f32<T>(r);
    const uint32_t xb = __float_as_uint(x);
    const float gap = __uint_as_float(xb & 0x7F800000u) * (((xb & 0x807FFFFFu) == 0u) ? 0.5f * gap_scale : gap_scale);
    const float off = gap >= 2.f ? gap * ((float)pos * pos_scale) : 0.f;
    return min(max(__float2int_rd(hiw - x * inv_w + off), 0), kBinCount - 1);
  }
};

template <typename T, int E>
__global__ void __launch_bounds__(kTopkThreads, 2) li_topk_bins_stream_kernel(LiDev p, const float* __restrict__ scores,
                                                                           int64_t ld) {
  constexpr int P2 = kTopkThreads * E;
  constexpr int NW = kTopkThreads / 32;
  __shared__ __align__(16) uint32_t hist[kBinCount];   // counts, then slot cursors
  __shared__ uint64_t buf[P2];                         // survivors by bin, any order inside a bin
  __shared__ uint16_t bbin[P2];                        // their bins
  __shared__ uint64_t side[kBinSide];                  // members of the crossing bin
  __shared__ uint32_t biglist[kBinBigList];
  __shared__ float2 part[NW];
  __shared__ uint32_t warp_tot[NW];
  __shared__ uint32_t counters[72];
  __shared__ uint32_t sh_bstar, sh_need, sh_cstar, sh_base, sh_side, sh_big;
  __shared__ unsigned long long sh_cut;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
  auto composite = [](uint32_t key16, uint32_t pos) -> uint64_t {
    return ((uint64_t)key16 << 32) | (uint64_t)(0xFFFFFFFFu - pos);
  };
  // a survivor's final slot is known: position and value go straight to the outputs
  auto emit = [&](uint32_t slot, uint64_t e) {
    oi[slot] = (int32_t)(0xFFFFFFFFu - (uint32_t)e);
    if (ov) ov[slot] = key16_bits<T>((uint32_t)(e >> 32));
  };

  // ---- 1. scale of the row from a sample of up to 512 scores spread over it
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist);
    h4[2 * tid] = make_uint4(0, 0, 0, 0);
    h4[2 * tid + 1] = make_uint4(0, 0, 0, 0);
  }
  if (tid < 72) counters[tid] = 0;
  if (tid == 0) { sh_bstar = kBinCount; sh_need = 0; sh_cstar = 0; sh_base = 0; sh_side = 0; sh_big = 0; sh_cut = 0ull; }
  BinScale<T> sc;
  {
    const int ns = min(n, kTopkThreads);
    const bool in = tid < ns;
    const int sp = n > kTopkThreads ? (int)(((int64_t)tid * n) >> 9) : tid;
    const float x = in ? round_io<T>(s[sp]) : 0.f;
    const float other = __shfl_xor_sync(0xffffffffu, x, 1);
    const float dv = (in && (tid ^ 1) < ns) ? fabsf(x - other) : 0.f;
    const float2 tot = block_sum2_f32(x, dv, part);
    const float mean = tot.x / (float)ns;
    const float sdev = 0.9f * (tot.y / (float)ns);
    float hi = mean + 5.f * sdev;
    float inv_w = sdev > 0.f ? (float)kBinCount / (8.f * sdev) : 0.f;
    if (!(fabsf(hi) <= 3.0e38f) || !(inv_w <= 3.0e38f)) { hi = 0.f; inv_w = 0.f; }
    constexpr int kMantBits = std::is_same<T, __half>::value ? 10 : 7;
    sc.hiw = hi * inv_w;
    sc.inv_w = inv_w;
    sc.gap_scale = inv_w * (1.f / (float)(1 << kMantBits));
    sc.pos_scale = (63.f / 64.f) / (float)n;
    if (!(fabsf(sc.hiw) <= 3.0e38f)) { sc.hiw = 0.f; sc.inv_w = 0.f; sc.gap_scale = 0.f; }
  }

  // ---- 2. first pass over the row: histogram (16-byte loads; rows start 16-byte aligned and are
  // padded to a multiple of 4 scores)
  for (int32_t pos0 = 4 * tid; pos0 < n; pos0 += 4 * kTopkThreads) {
    const float4 v = *reinterpret_cast<const float4*>(s + pos0);
    const float xs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (pos0 + u < n) atomicAdd(&hist[sc.bin(from_f32<T>(xs[u]), (uint32_t)(pos0 + u))], 1u);
  }
  __syncthreads();

  // ---- 3. slot at which every bin starts; the bin in which the count crosses K
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist);
    uint4 a = h4[2 * tid], c = h4[2 * tid + 1];
    uint32_t cnt[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
    uint32_t sum = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) sum += cnt[q];
    uint32_t inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    uint32_t run = inc - sum;
    {
      const uint32_t wt = warp_tot[lane & (NW - 1)];
      uint32_t winc = wt;
#pragma unroll
      for (int o = 1; o < NW; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
        if ((lane & (NW - 1)) >= o) winc += t;
      }
      run += __shfl_sync(0xffffffffu, winc - wt, warp);
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint32_t c0 = cnt[q];
      if (run < (uint32_t)K && (uint32_t)K <= run + c0) {
        sh_bstar = 8 * tid + q; sh_base = run; sh_need = (uint32_t)K - run; sh_cstar = c0;
      }
      cnt[q] = run;
      run += c0;
    }
    h4[2 * tid] = make_uint4(cnt[0], cnt[1], cnt[2], cnt[3]);
    h4[2 * tid + 1] = make_uint4(cnt[4], cnt[5], cnt[6], cnt[7]);
  }
  __syncthreads();
  const uint32_t bstar = sh_bstar, need = sh_need, cstar = sh_cstar, base_star = sh_base;
  const bool side_cut = cstar <= (uint32_t)kBinSide;

  // ---- 4. a large crossing bin is cut by bisection on the composite (one pass over the row per step)
  uint64_t cut = 0ull;
  if (bstar < (uint32_t)kBinCount && !side_cut) {
    uint64_t lo = 1ull, hi_c = 0xFFFFFFFFFFFFull;
    int slot = 0;
#pragma unroll 1
    for (int it = 0; it < 64 && lo < hi_c; ++it, ++slot) {
      const uint64_t mid = lo + ((hi_c - lo) >> 1) + ((hi_c - lo) & 1ull);
      uint32_t c = 0;
      for (int32_t pos = tid; pos < n; pos += kTopkThreads) {
        const T r = from_f32<T>(s[pos]);
        c += (uint32_t)sc.bin(r, (uint32_t)pos) == bstar && composite(rank_key_of<T>(r), (uint32_t)pos) >= mid;
      }
      const uint32_t total = block_count(c, &counters[slot]);
      if (total >= need) lo = mid; else hi_c = mid - 1ull;
    }
    cut = lo;
  }

  // ---- 5. second pass over the row: survivors into their bin's slot range
  for (int32_t pos0 = 4 * tid; pos0 < n; pos0 += 4 * kTopkThreads) {
    const float4 v = *reinterpret_cast<const float4*>(s + pos0);
    const float xs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t pos = (uint32_t)(pos0 + u);
      if ((int32_t)pos >= n) continue;
      const T r = from_f32<T>(xs[u]);
      const uint32_t b = (uint32_t)sc.bin(r, pos);
      if (b > bstar) continue;
      const uint64_t comp = composite(rank_key_of<T>(r), pos);
      if (b < bstar || (!side_cut && comp >= cut)) {
        const uint32_t slot = atomicAdd(&hist[b], 1u);
        if (slot < (uint32_t)P2) { buf[slot] = comp; bbin[slot] = (uint16_t)b; }
      } else if (side_cut) {
        side[atomicAdd(&sh_side, 1u)] = comp;
      }
    }
  }
  __syncthreads();

  // ---- 6. order inside each bin
  {
#pragma unroll
    for (int r = 0; r < E; ++r) {
      const int e = r * kTopkThreads + tid;
      if (e < nsel && (!side_cut || (uint32_t)e < base_star || bstar == (uint32_t)kBinCount)) {
        const uint64_t mine = buf[e];
        const uint32_t b = bbin[e];
        const uint32_t st = b ? hist[b - 1] : 0u;
        const uint32_t cn = min(hist[b], (uint32_t)nsel) - st;
        if (cn > (uint32_t)kBinSmall) {
          if ((uint32_t)e == st) {
            const uint32_t i = atomicAdd(&sh_big, 1u);
            if (i < (uint32_t)kBinBigList) biglist[i] = b;
          }
        } else {
          uint32_t rank = 0;
          for (uint32_t q = st; q < st + cn; ++q) rank += buf[q] > mine;
          emit(st + rank, mine);
        }
      }
    }
    if (side_cut && (uint32_t)tid < cstar) {
      const uint64_t m = side[tid];
      uint32_t rank = 0;
      for (uint32_t q = 0; q < cstar; ++q) rank += side[q] > m;
      if (rank < need) emit(base_star + rank, m);
    }
  }
  __syncthreads();
  {
    const uint32_t nbig = min(sh_big, (uint32_t)kBinBigList);
    for (uint32_t i = 0; i < nbig; ++i) {
      const uint32_t b = biglist[i];
      const uint32_t st = b ? hist[b - 1] : 0u;
      const uint32_t en = min(hist[b], (uint32_t)nsel);
      const bool shared_bin = en - st > 256u;
      if (!shared_bin && (i % NW) != (uint32_t)warp) continue;
      for (uint32_t m0 = st + (shared_bin ? 32u * warp : 0u); m0 < en; m0 += shared_bin ? 32u * NW : 32u) {
        const uint32_t m = m0 + lane;
        const uint64_t mine = m < en ? buf[m] : 0ull;
        uint32_t rank = 0;
        for (uint32_t q = st; q < en; ++q) rank += buf[q] > mine;
        if (m < en) emit(st + rank, mine);
      }
    }
  }

  // ---- 7. unused slots
  for (int i = nsel + tid; i < K; i += kTopkThreads) {
    oi[i] = -1;
    if (ov) ov[i] = from_f32<T>(0.f);
  }
}

}  // namespace dsa