// Lightning-indexer score kernel on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Shape served: 16..64 query heads sharing one key head, head dim 128, bf16 or fp16; BSND, TND or paged
// keys (block size 16/32/64 or a multiple of 128: a 128-key tile is then one or a few whole-block
// TMA loads whose rows come from the block table; an absent block loads as zeros through an
// out-of-range row coordinate).
//
// GEMM orientation: KEYS sit on the MMA M axis (128 keys = 128 TMEM lanes) and (token, head)
// pairs on the N axis (4 tokens x 64 heads = 256 columns), so that after a TMEM load every
// thread owns one key and the ReLU * weight * head-sum epilogue is thread-local.
//
// One CTA works on items of 8 consecutive query rows of one sequence: their Q (8 x 64 x 128,
// 128 KB) stays in shared memory while 128-key tiles stream through a 3-stage TMA ring.  Each key
// tile feeds two accumulators (rows 0-3 and rows 4-7, 256 TMEM columns each), which double-buffer
// the epilogue against the MMAs.  Tiles beyond the causal limit of the item's last row are
// skipped; the diagonal tile is masked in the epilogue.  Items are statically spread over a
// persistent grid in snake order of decreasing work.  When there are too few row groups to fill
// the GPU (decode: a few rows against very long key sequences) an item is a row group times a
// chunk of key tiles, and groups of at most 4 rows use only the first accumulator.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..9
// epilogue (TMEM lane quarter = warp % 4, column half = (warp - 2) / 4).
#pragma once

#include <atomic>
#include <mutex>

#include "li_score_simt.cuh"
#include "ptx_sm100.cuh"

namespace dsa {

constexpr int kLiTok = 8;        // query rows per item
constexpr int kLiHalf = 4;       // query rows per accumulator
constexpr int kLiHeads = 64;
constexpr int kLiDim = 128;
constexpr int kLiKeys = 128;     // keys per tile
constexpr int kLiStages = 3;      // key stages behind the 128 KB of Q
constexpr int kLiMaxStages = 5;   // two more in the unused half of the Q buffer when no item has more than 4 rows
constexpr int kLiThreads = 320;
constexpr int kLiEpiWarps = 8;

constexpr uint32_t kLiQBlock = 256 * 128;                 // one 64-column block of one half: 256 rows x 128 B
constexpr uint32_t kLiQBytes = 4 * kLiQBlock;             // 2 halves x 2 column blocks = 128 KB
constexpr uint32_t kLiKBlock = kLiKeys * 128;             // 128 rows x 128 B
constexpr uint32_t kLiKStage = 2 * kLiKBlock;             // 32 KB
constexpr uint32_t kLiOffK = kLiQBytes;
constexpr uint32_t kLiOffW = kLiOffK + kLiStages * kLiKStage;
constexpr uint32_t kLiOffBar = kLiOffW + kLiTok * kLiHeads * 4;
constexpr int kLiDenseGroups = 128;   // most row groups of the dense chunked mode (its table sits behind the barriers)
constexpr uint32_t kLiOffCum = kLiOffBar + 256;
constexpr uint32_t kLiSmemBytes = kLiOffCum + (kLiDenseGroups + 2) * 4;
// Byte offset of key stage s: stages 3 and 4 live in the second half of the Q buffer.
__host__ __device__ constexpr uint32_t li_stage_off(uint32_t s) {
  return s < (uint32_t)kLiStages ? kLiOffK + s * kLiKStage : 2 * kLiQBlock + (s - kLiStages) * kLiKStage;
}

struct LiSm100Args {
  LiDev p;
  float* scores;
  int64_t ld;
  int32_t* status;        // device status word (workspace header)
  int32_t groups_per_seq; // ceil(s1 / 8)
  int32_t groups;         // row groups (an upper bound for TND)
  int32_t items;          // groups * nchunks
  int32_t nchunks;        // key chunks per row group (1 = a group takes all its key tiles)
  int32_t chunk_tiles;    // key tiles per chunk
  int32_t stages;         // key stages in use: 3, or 5 when no row group has more than 4 rows
  int32_t sub_rows;       // key rows per TMA load: 128, or the block size of a paged cache if smaller
  int32_t krow_oob;       // a row coordinate past the key tensor (loads as zeros)
  uint32_t idesc;         // M=128, N=256: four rows per accumulator
  uint32_t idesc_n128;    // M=128, N=128: row groups of at most two rows
  int32_t dense;          // chunked mode: items are only the chunks that hold keys (see li_dense_setup)
};

// One work item: up to 8 consecutive query rows of one sequence.
struct LiItem {
  int32_t row0;    // first global query row (BSND: b * s1 + pos, TND: token index); -1 = no such item
  int32_t nrows;   // 1..8 rows that exist in the sequence
  int32_t b;       // sequence
  int32_t chunk;   // key chunk
  int64_t krow0;   // first key row of the sequence in the key tensor (not paged)
};
// Item i -> rows.  BSND: sequences interleaved, later row groups first (under the causal mask they
// see more keys, so item 0 is the most work).  TND: sequences in order (their group counts are
// only known on the device), later groups first inside each sequence.
__device__ __forceinline__ LiItem li_group(const LiSm100Args& a, int32_t i) {
  LiItem it;
  it.row0 = -1; it.nrows = 0; it.krow0 = 0; it.b = 0; it.chunk = 0;
  const SeqDesc& s = a.p.seq;
  int32_t b, pos0, len_q, start_q;
  if (s.layout_q == DSA_LAYOUT_TND) {
    int32_t acc = 0, prev = 0;
    for (b = 0; b < s.batch; ++b) {
      const int32_t end = s.seq_q[b];
      const int32_t g = (end - prev + kLiTok - 1) / kLiTok;
      if (i < acc + g) {
        start_q = prev; len_q = end - prev;
        pos0 = (g - 1 - (i - acc)) * kLiTok;
        break;
      }
      acc += g; prev = end;
    }
    if (b >= s.batch) return it;
  } else {
    b = i % s.batch;
    pos0 = (a.groups_per_seq - 1 - i / s.batch) * kLiTok;
    start_q = b * s.s1; len_q = s.s1;
  }
  it.row0 = start_q + pos0;
  it.nrows = min(kLiTok, len_q - pos0);
  it.b = b;
  it.krow0 = row_info(s, it.row0).key_base;
  return it;
}
// `cum` (shared memory, dense mode only): cum[g] = chunks with keys of the row groups before g,
// cum[groups] = their total, cum[kLiDenseGroups + 1] = key tiles per chunk.
template <bool kDense>
__device__ __forceinline__ LiItem li_item(const LiSm100Args& a, int32_t i, const int32_t* cum) {
  if constexpr (kDense) {
    if (i >= cum[a.groups]) {
      LiItem none;
      none.row0 = -1; none.nrows = 0; none.krow0 = 0; none.b = 0; none.chunk = 0;
      return none;
    }
    int32_t lo = 0, hi = a.groups;          // largest g with cum[g] <= i
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (cum[mid] <= i) lo = mid; else hi = mid;
    }
    LiItem it = li_group(a, lo);
    it.chunk = i - cum[lo];
    return it;
  }
  // chunk-major: the first chunks exist for every sequence, later ones only for the long sequences,
  // so work decreases with the item number as the snake order assumes
  const int32_t chunk = i / a.groups;
  LiItem it = li_group(a, i - chunk * a.groups);
  it.chunk = chunk;
  return it;
}
// j-th item of CTA c in snake order over a persistent grid of g CTAs (-1 when exhausted).
__device__ __forceinline__ int32_t li_item_of(int32_t c, int32_t g, int32_t j, int32_t items) {
  const int32_t i = (j & 1) ? (j * g + (g - 1 - c)) : (j * g + c);
  return i < items ? i : -1;
}
// Visible key count of each of the item's rows and the item's key tiles [t0, t1); false if none.
template <bool kDense>
__device__ __forceinline__ bool li_item_range(const LiSm100Args& a, const LiItem& it, int32_t* vis, int32_t* t0,
                                              int32_t* t1, const int32_t* cum) {
  int32_t mx = 0;
#pragma unroll
  for (int t = 0; t < kLiTok; ++t) {
    int32_t v = 0;
    if (t < it.nrows) v = row_info(a.p.seq, it.row0 + t).visible;
    if (vis) vis[t] = v;
    mx = max(mx, v);
  }
  const int32_t tiles = (mx + kLiKeys - 1) / kLiKeys;
  const int32_t ct = kDense ? cum[kLiDenseGroups + 1] : a.chunk_tiles;
  *t0 = it.chunk * ct;
  *t1 = min(tiles, *t0 + ct);
  return *t1 > *t0;
}

// kDense: chunked mode over the list of chunks that hold keys (decode); compiled apart so that the
// prefill instantiation carries none of it.
template <bool kDense>
__global__ void __launch_bounds__(kLiThreads, 1)
li_score_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const LiSm100Args a) {
  extern __shared__ __align__(1024) unsigned char li_smem[];
  unsigned char* q_s = li_smem;
  float* w_s = reinterpret_cast<float*>(li_smem + kLiOffW);
  uint64_t* bars = reinterpret_cast<uint64_t*>(li_smem + kLiOffBar);
  uint64_t* full = bars;            // [5] TMA -> MMA
  uint64_t* empty = bars + 5;       // [5] MMA -> TMA
  uint64_t* qfull = bars + 10;
  uint64_t* qempty = bars + 11;
  uint64_t* tfull = bars + 12;      // [2] MMA -> epilogue
  uint64_t* tempty = bars + 14;     // [2] epilogue -> MMA
  uint64_t* wbar = bars + 16;       // epilogue-internal rendezvous around the weight staging
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 18);
  int32_t* cum_s = reinterpret_cast<int32_t*>(li_smem + kLiOffCum);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t cta = blockIdx.x, grid = gridDim.x;

  if ((ptx::smem_u32(li_smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicExch(a.status, 2);
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < kLiMaxStages; ++i) { ptx::mbar_init(&full[i], 1); ptx::mbar_init(&empty[i], 1); }
    ptx::mbar_init(qfull, 1);
    ptx::mbar_init(qempty, 1);
    for (int i = 0; i < 2; ++i) { ptx::mbar_init(&tfull[i], 1); ptx::mbar_init(&tempty[i], kLiEpiWarps); }
    ptx::mbar_init(wbar, kLiEpiWarps * 32);
    *abort_flag = 0;
    ptx::mbar_fence_init();
  }
  if (a.p.n1 != kLiHeads) {
    // fewer than 64 heads: the spare rows of every token's slot in the Q buffer must read as zero
    for (uint32_t i = threadIdx.x; i < kLiQBytes / 16; i += kLiThreads)
      reinterpret_cast<uint4*>(li_smem)[i] = make_uint4(0, 0, 0, 0);
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  if constexpr (kDense) {
    // li_dense_setup: key tiles of every row group (every CTA builds the same list)
    for (int g = threadIdx.x; g < a.groups; g += kLiThreads) {
      const LiItem it = li_group(a, g);
      int32_t mx = 0;
      if (it.row0 >= 0)
        for (int t = 0; t < it.nrows; ++t) mx = max(mx, row_info(a.p.seq, it.row0 + t).visible);
      cum_s[g + 1] = (mx + kLiKeys - 1) / kLiKeys;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if constexpr (kDense) {
    // chunk size: about eight chunks of real work per CTA, at least 8 tiles each; then the running
    // count of chunks per group.  The static round-robin over this list leaves the CTAs within one
    // chunk of each other, where the (chunk, group) grid leaves them with whatever mix of full,
    // partial and empty chunks the sequence lengths produce.
    if (threadIdx.x == 0) {
      int64_t total = 0;
      for (int g = 0; g < a.groups; ++g) total += cum_s[g + 1];
      int64_t ct = (total + 8ll * grid - 1) / (8ll * grid);
      if (ct < 8) ct = 8;
      int32_t acc = 0;
      cum_s[0] = 0;
      for (int g = 0; g < a.groups; ++g) {
        acc += (int32_t)((cum_s[g + 1] + ct - 1) / ct);
        cum_s[g + 1] = acc;
      }
      cum_s[kLiDenseGroups + 1] = (int32_t)ct;
    }
    __syncthreads();
  }
  const uint32_t tmem = *tmem_slot;
  // Q of an item -> shared memory.  64 heads: one 256-row box per half and column block.  Fewer
  // heads (16..63): one box of n1 rows per token into the token's 64-row slot; the slot's other
  // rows were zeroed once at kernel start and are never written, and their weights are zero.
  const int32_t n1 = a.p.n1;
  auto q_bytes = [&](int nh) -> uint32_t {
    return n1 == kLiHeads ? (uint32_t)nh * 2u * kLiQBlock : (uint32_t)nh * kLiHalf * 2u * (uint32_t)n1 * 128u;
  };
  auto load_q = [&](int32_t row0, int nh) {
    if (n1 == kLiHeads) {
      const int32_t qrow = row0 * kLiHeads;
      for (int h = 0; h < nh; ++h)
#pragma unroll
        for (int c = 0; c < 2; ++c)
          ptx::tma_load_2d(q_s + (h * 2 + c) * kLiQBlock, &tmap_q, qfull, c * 64, qrow + h * kLiHalf * kLiHeads);
    } else {
      for (int t = 0; t < nh * kLiHalf; ++t)
#pragma unroll
        for (int c = 0; c < 2; ++c)
          ptx::tma_load_2d(q_s + ((t / kLiHalf) * 2 + c) * kLiQBlock + (t % kLiHalf) * kLiHeads * 128, &tmap_q, qfull,
                           c * 64, (row0 + t) * n1);
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // Lane 0 issues; the other lanes only help with the block table of a paged cache (lane u looks
    // up the u-th whole-block load of a tile, one tile ahead of its use).
    if (lane == 0) {
      ptx::prefetch_tmap(&tmap_q);
      ptx::prefetch_tmap(&tmap_k);
    }
    const SeqDesc& sq = a.p.seq;
    const bool paged = sq.layout_k == DSA_LAYOUT_PA_BSND;
    const int nsub = kLiKeys / a.sub_rows;
    uint32_t n_item = 0, s = 0, use = 0;   // ring position: stage and how often the ring went round
    const uint32_t stages = a.stages;
    bool ok = true;
    if (!paged) {
      // contiguous keys: one thread does everything
      if (lane == 0) {
        for (int32_t j = 0; ok; ++j) {
          const int32_t it = li_item_of(cta, grid, j, a.items);
          if (it < 0) break;
          const LiItem item = li_item<kDense>(a, it, cum_s);
          if (item.row0 < 0) continue;
          int32_t t0, t1;
          if (!li_item_range<kDense>(a, item, nullptr, &t0, &t1, cum_s)) continue;
          const int nh = item.nrows > kLiHalf ? 2 : 1;
          ok = ptx::mbar_wait(qempty, (n_item & 1) ^ 1, abort_flag);
          if (!ok) break;
          ptx::mbar_arrive_expect_tx(qfull, q_bytes(nh));
          load_q(item.row0, nh);
          ++n_item;
          const int32_t krow0 = (int32_t)item.krow0;
          for (int32_t t = t0; t < t1; ++t) {
            ok = ptx::mbar_wait(&empty[s], (use & 1) ^ 1, abort_flag);
            if (!ok) break;
            ptx::mbar_arrive_expect_tx(&full[s], kLiKStage);
            unsigned char* dst = li_smem + li_stage_off(s);
            ptx::tma_load_2d(dst, &tmap_k, &full[s], 0, krow0 + t * kLiKeys);
            ptx::tma_load_2d(dst + kLiKBlock, &tmap_k, &full[s], 64, krow0 + t * kLiKeys);
            if (++s == stages) { s = 0; ++use; }
          }
        }
      }
    } else
    for (int32_t j = 0; ok; ++j) {
      const int32_t it = li_item_of(cta, grid, j, a.items);
      if (it < 0) break;
      const LiItem item = li_item<kDense>(a, it, cum_s);
      if (item.row0 < 0) continue;
      int32_t t0, t1;
      if (!li_item_range<kDense>(a, item, nullptr, &t0, &t1, cum_s)) continue;
      const int nh = item.nrows > kLiHalf ? 2 : 1;
      if (lane == 0) {
        ok = ptx::mbar_wait(qempty, (n_item & 1) ^ 1, abort_flag);
        if (ok) {
          ptx::mbar_arrive_expect_tx(qfull, q_bytes(nh));
          load_q(item.row0, nh);
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      if (!ok) break;
      ++n_item;
      // first key row of this lane's load of tile t
      auto sub_row = [&](int32_t t) -> int32_t {
        const int32_t p = t * kLiKeys + lane * a.sub_rows;
        if (!paged) return (int32_t)item.krow0 + p;
        const int32_t bi = p / sq.block_size;
        if (lane >= nsub || bi >= sq.max_blocks) return a.krow_oob;
        const int32_t blk = sq.block_table[(int64_t)item.b * sq.max_blocks + bi];
        if (blk < 0) return a.krow_oob;
        const int64_t r = (int64_t)blk * sq.block_size + (p - bi * sq.block_size);
        return r < (int64_t)a.krow_oob ? (int32_t)r : a.krow_oob;
      };
      int32_t cur = sub_row(t0);
      for (int32_t t = t0; t < t1; ++t) {
        const int32_t nxt = (t + 1 < t1) ? sub_row(t + 1) : 0;
        if (lane == 0) ok = ptx::mbar_wait(&empty[s], (use & 1) ^ 1, abort_flag);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        if (lane == 0) ptx::mbar_arrive_expect_tx(&full[s], kLiKStage);
        for (int u = 0; u < nsub; ++u) {
          const int32_t r = __shfl_sync(0xffffffffu, cur, u);
          if (lane == 0) {
            unsigned char* dst = li_smem + li_stage_off(s) + u * a.sub_rows * 128;
            ptx::tma_load_2d(dst, &tmap_k, &full[s], 0, r);
            ptx::tma_load_2d(dst + kLiKBlock, &tmap_k, &full[s], 64, r);
          }
        }
        cur = nxt;
        if (++s == stages) { s = 0; ++use; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      uint32_t n_item = 0, s = 0, use = 0, n_use0 = 0, n_use1 = 0;   // ring position; uses of each accumulator
      const uint32_t stages = a.stages;
      bool ok = true;
      const uint32_t q_addr = ptx::smem_u32(q_s), smem_base = ptx::smem_u32(li_smem);
      for (int32_t j = 0; ok; ++j) {
        const int32_t it = li_item_of(cta, grid, j, a.items);
        if (it < 0) break;
        const LiItem item = li_item<kDense>(a, it, cum_s);
        if (item.row0 < 0) continue;
        int32_t t0, t1;
        if (!li_item_range<kDense>(a, item, nullptr, &t0, &t1, cum_s)) continue;
        const int nh = item.nrows > kLiHalf ? 2 : 1;
        const uint32_t idesc = item.nrows <= 2 ? a.idesc_n128 : a.idesc;
        ok = ptx::mbar_wait(qfull, n_item & 1, abort_flag);
        if (!ok) break;
        ++n_item;
        for (int32_t t = t0; t < t1 && ok; ++t) {
          ok = ptx::mbar_wait(&full[s], use & 1, abort_flag);
          if (!ok) break;
          const uint32_t k_addr = smem_base + li_stage_off(s);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (h >= nh) break;
            // row half h of the item goes to accumulator `acc`: a group of at most four rows has one
            // half only and alternates between the two accumulators from tile to tile, so that its
            // epilogue still overlaps the next tile's MMAs
            const int acc = nh == 2 ? h : (int)(n_use0 + n_use1) & 1;
            ok = ptx::mbar_wait(&tempty[acc], ((acc ? n_use1 : n_use0) & 1) ^ 1, abort_flag);
            if (!ok) break;
            ptx::tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < kLiDim / 16; ++ks) {
              const uint32_t ka = k_addr + (ks >> 2) * kLiKBlock + (ks & 3) * 32;
              const uint32_t qa = q_addr + h * 2 * kLiQBlock + (ks >> 2) * kLiQBlock + (ks & 3) * 32;
              ptx::mma_ss(tmem + acc * 256, ptx::desc_kmajor_sw128(ka), ptx::desc_kmajor_sw128(qa), idesc, ks > 0);
            }
            ptx::mma_commit(&tfull[acc]);
            if (acc) ++n_use1; else ++n_use0;
          }
          if (!ok) break;
          ptx::mma_commit(&empty[s]);
          if (++s == stages) { s = 0; ++use; }
        }
        if (ok) ptx::mma_commit(qempty);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps)
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int chalf = ew >> 2;
    const int et = threadIdx.x - 64;  // 0..255
    uint32_t n_tile = 0, n_use0 = 0, n_use1 = 0, n_sync = 0;
    bool ok = true;
    for (int32_t j = 0; ok; ++j) {
      const int32_t it = li_item_of(cta, grid, j, a.items);
      if (it < 0) break;
      int32_t vis[kLiTok];
      const LiItem item = li_item<kDense>(a, it, cum_s);
      if (item.row0 < 0) continue;
      int32_t t0, t1;
      if (!li_item_range<kDense>(a, item, vis, &t0, &t1, cum_s)) continue;
      const int nh = item.nrows > kLiHalf ? 2 : 1;
      const int32_t row0 = item.row0;
      // weights of the item's 8 rows -> shared memory (rows past the sequence end read as zero)
      // (rendezvous through an mbarrier so that even this wait is bounded)
      ptx::mbar_arrive(wbar);
      ok = ptx::mbar_wait(wbar, n_sync++ & 1, abort_flag);
      if (!ok) break;
      for (int i = et; i < kLiTok * kLiHeads; i += 256) {
        const int t = i / kLiHeads;
        const int hh = i - t * kLiHeads;
        w_s[i] = (t < item.nrows && hh < n1) ? load_weight(a.p.weights, a.p.dtype_w, (int64_t)(row0 + t) * n1 + hh) : 0.f;
      }
      ptx::mbar_arrive(wbar);
      ok = ptx::mbar_wait(wbar, n_sync++ & 1, abort_flag);
      if (!ok) break;
      for (int32_t t = t0; t < t1 && ok; ++t, ++n_tile) {
        const int32_t pos = t * kLiKeys + quarter * 32 + lane;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h >= nh) break;
          const int acc = nh == 2 ? h : (int)(n_use0 + n_use1) & 1;   // as in the MMA issuer
          ok = ptx::mbar_wait(&tfull[acc], (acc ? n_use1 : n_use0) & 1, abort_flag);
          if (!ok) break;
          if (acc) ++n_use1; else ++n_use0;
          ptx::tc_fence_after();
          const int tok0 = h * kLiHalf + chalf * 2;
          // (rows that do not exist are computed as well and dropped by the `vis` test below: making
          // the loads conditional cost the full-size case 45 %)
          uint32_t r0[64], r1[64];
          const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + acc * 256 + chalf * 128;
          ptx::tmem_ld_x32(taddr, r0);
          ptx::tmem_ld_x32(taddr + 32, r0 + 32);
          ptx::tmem_ld_x32(taddr + 64, r1);
          ptx::tmem_ld_x32(taddr + 96, r1 + 32);
          ptx::tmem_ld_wait();
          // the accumulator is in registers: hand the TMEM buffer back before doing the math
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&tempty[acc]);
          // the arithmetic (not the loads above) is skipped for rows that do not exist; in decode
          // that is half of the epilogue warps
          if (tok0 < item.nrows) {
            const float* w0 = w_s + tok0 * kLiHeads;
            const float* w1 = w0 + kLiHeads;
            float s0a = 0.f, s0b = 0.f, s1a = 0.f, s1b = 0.f;
#pragma unroll
            for (int g = 0; g < kLiHeads; g += 2) {
              s0a = fmaf(fmaxf(__uint_as_float(r0[g]), 0.f), w0[g], s0a);
              s0b = fmaf(fmaxf(__uint_as_float(r0[g + 1]), 0.f), w0[g + 1], s0b);
              s1a = fmaf(fmaxf(__uint_as_float(r1[g]), 0.f), w1[g], s1a);
              s1b = fmaf(fmaxf(__uint_as_float(r1[g + 1]), 0.f), w1[g + 1], s1b);
            }
            if (pos < vis[tok0]) a.scores[(int64_t)(row0 + tok0) * a.ld + pos] = s0a + s0b + 0.f;
            if (pos < vis[tok0 + 1]) a.scores[(int64_t)(row0 + tok0 + 1) * a.ld + pos] = s1a + s1b + 0.f;
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) {
    // a bounded wait gave up: give copies and MMAs still in flight time to land before the
    // shared and tensor memory they target is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(a.status, 1);
}

// Host side: eligibility, tensor maps, launch.
inline bool li_sm100_eligible(const DsaLiParams* p) {
  if (p->layout_k == DSA_LAYOUT_PA_BSND) {
    // a 128-key tile must be whole blocks, or lie inside one
    const int bs = p->block_size;
    if (!(bs == 16 || bs == 32 || bs == 64 || (bs >= 128 && bs % 128 == 0))) return false;
    if (p->block_table == nullptr || p->max_blocks < 1) return false;
  }
  // 16..63 heads (a tensor-parallel shard) run with zero rows and zero weights in the spare slots
  if (p->n1 < 16 || p->n1 > kLiHeads || p->n2 != 1 || p->d != kLiDim) return false;
  if (p->s1 < 1 || p->s2 < 1) return false;
  if (((uintptr_t)p->query & 15u) || ((uintptr_t)p->key & 15u)) return false;
  const int64_t rows = p->layout_q == DSA_LAYOUT_TND ? (int64_t)p->s1 : (int64_t)p->batch * p->s1;
  if (rows * kLiHeads >= (1ll << 31) || p->key_rows < 1 || p->key_rows >= (1ll << 31)) return false;
  if (p->layout_q == DSA_LAYOUT_BSND && p->seq_q_cumulative) return false;
  return true;
}

inline int li_sm100_launch(const DsaLiParams* p, const LiDev& d, float* scores, int64_t ld, int32_t* status,
                           cudaStream_t st) {
  // SM count per device, set up once per device (safe from several host threads)
  static std::atomic<int> sm_count[64];
  static std::mutex setup_lock;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DSA_ERR_CUDA;
  if (sm_count[dev].load(std::memory_order_acquire) == 0) {
    std::lock_guard<std::mutex> g(setup_lock);
    if (sm_count[dev].load(std::memory_order_relaxed) == 0) {
      int n = 0;
      if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) return DSA_ERR_CUDA;
      if (cudaFuncSetAttribute(li_score_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)kLiSmemBytes) != cudaSuccess ||
          cudaFuncSetAttribute(li_score_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)kLiSmemBytes) != cudaSuccess)
        return DSA_ERR_CUDA;
      sm_count[dev].store(n, std::memory_order_release);
    }
  }
  const int sms = sm_count[dev].load(std::memory_order_relaxed);
  const bool bf16 = p->dtype_qk == DSA_DTYPE_BF16;
  CUtensorMap tq, tk;
  const bool tnd = p->layout_q == DSA_LAYOUT_TND;
  const uint64_t qrows = tnd ? (uint64_t)p->s1 : (uint64_t)p->batch * p->s1;
  if (!make_tmap_2d_16bit(&tq, p->query, qrows * p->n1, kLiDim, kLiDim * 2, p->n1 == kLiHeads ? 256 : p->n1, 64, bf16))
    return DSA_ERR_CUDA;
  const bool paged = p->layout_k == DSA_LAYOUT_PA_BSND;
  const int sub_rows = (paged && p->block_size < kLiKeys) ? p->block_size : kLiKeys;
  if (!make_tmap_2d_16bit(&tk, p->key, (uint64_t)p->key_rows, kLiDim, kLiDim * 2, sub_rows, 64, bf16))
    return DSA_ERR_CUDA;
  LiSm100Args a;
  a.p = d;
  a.scores = scores;
  a.ld = ld;
  a.status = status;
  a.groups_per_seq = (p->s1 + kLiTok - 1) / kLiTok;
  // TND: the group count of a sequence is only known on the device; this is an upper bound and
  // li_item() reports the surplus as empty
  const int32_t groups = tnd ? (p->s1 + kLiTok - 1) / kLiTok + p->batch : p->batch * a.groups_per_seq;
  // few row groups (decode): split each group's key tiles into chunks so that every SM gets work
  const int64_t keys_max = paged ? (int64_t)p->max_blocks * p->block_size : (int64_t)p->s2;
  const int32_t tiles_max = (int32_t)((keys_max + kLiKeys - 1) / kLiKeys);
  a.nchunks = 1;
  a.chunk_tiles = tiles_max > 0 ? tiles_max : 1;
  if (groups < 2 * sms && tiles_max > 1) {
    // static assignment: many small chunks (>= 8 tiles each) even out sequences of unequal length;
    // about eight items per SM measured best on 64 sequences of 16K-64K keys (28 tiles per chunk)
    int32_t want = (8 * sms + groups - 1) / groups;
    if (want > tiles_max) want = tiles_max;
    a.chunk_tiles = (tiles_max + want - 1) / want;
    if (a.chunk_tiles < 8) a.chunk_tiles = tiles_max < 8 ? tiles_max : 8;
    a.nchunks = (tiles_max + a.chunk_tiles - 1) / a.chunk_tiles;
  }
  a.groups = groups;
  a.stages = (!tnd && p->s1 <= kLiHalf) ? kLiMaxStages : kLiStages;
  a.items = groups * a.nchunks;
  a.sub_rows = sub_rows;
  a.krow_oob = (int32_t)p->key_rows;
  a.idesc = ptx::idesc_f16(bf16 ? 1u : 0u, 128, 256, 0, 0);
  a.idesc_n128 = ptx::idesc_f16(bf16 ? 1u : 0u, 128, 128, 0, 0);
  // chunked mode with few enough row groups: the kernel lists the chunks that hold keys itself
  // (the lengths live on the device) and sizes them so that every CTA gets about eight
  a.dense = (a.nchunks > 1 && groups <= kLiDenseGroups) ? 1 : 0;
  if (a.dense) a.items = groups * ((tiles_max + 7) / 8);      // upper bound: chunks are at least 8 tiles
  const int grid = a.items < sms ? a.items : sms;
  if (a.dense) li_score_sm100_kernel<true><<<grid, kLiThreads, kLiSmemBytes, st>>>(tq, tk, a);
  else li_score_sm100_kernel<false><<<grid, kLiThreads, kLiSmemBytes, st>>>(tq, tk, a);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  count_launch();
  return DSA_OK;
}

}  // namespace dsa
