// Sparse flash attention forward on tcgen05 tensor cores for the MLA-absorb production shape:
// 128 query heads, D = 512 (+64 rope), one KV head, any layout, token- or block-wise indices.
// 16..127 heads (a tensor-parallel shard of the 128) run the same code with the spare accumulator
// lanes carrying zero queries; few query rows (decode at small batch) are split along their keys
// into parts whose partial results a small kernel merges.
//
// Why a 2-CTA cluster per query token.  One token's accumulator O[128 heads x 512] in fp32 is the
// whole tensor memory of an SM (128 lanes x 512 columns) and its Q[128 x 576] is 147 KB of shared
// memory, so a single SM cannot hold O, the scores and a deep enough ring of gathered KV rows.
// The two CTAs of a cluster split the FEATURE axis instead of the heads (which would halve the MMA
// M dimension and with it the tensor throughput):
//     CTA 0: nope columns   0..255 + the 64 rope columns  (320 dims of QK^T, value columns   0..255)
//     CTA 1: nope columns 256..511                         (256 dims of QK^T, value columns 256..511)
// Each CTA gathers only its own half of every selected KV row (TMA tile::gather4 into the
// 128-byte-swizzled MMA layout, 4-stage ring), computes a PARTIAL S = Q_c K_c^T for all 128 heads,
// sends it to its peer through distributed shared memory, adds the peer's partial, runs the
// softmax (both CTAs hold the same full S, so no running-max exchange is needed) and accumulates
// O_c = P V_c with V_c = the nope columns it already holds.  Every MMA is a full-rate 128-row
// cta_group::1 instruction, every KV byte crosses L2->SM once, and no flop is duplicated except
// the softmax arithmetic.
//
// Gather issue rate (measured with in-kernel cycle counters and a micro-probe on a B200): one warp
// issues one 512-byte gather4 load per ~67 cycles (~7.5 B/clk) however its lanes are arranged, a
// 16-byte cp.async warp instruction costs ~115 cycles (~4.4 B/clk per warp), and both scale
// linearly with the number of issuing warps (6 warps: ~42 B/clk).  A tile's 80 loads issued from a
// single warp took ~6100 cycles against ~1150 cycles of MMA work, so the loads of every tile are
// spread over ten producer warps (under load, next to the MMAs and the
// bulk copies, a producer warp needs ~170 cycles per load).
//
// A small pre-pass kernel turns every row's sparse indices into a front-packed list of physical KV
// rows plus a count (block-wise ids expanded, -1 / out-of-window entries dropped, paged positions
// translated through the block table), so the hot loop does no index arithmetic.
//
// Tensor memory per CTA (512 columns): O 0..255 | Q (bf16 pairs, MMA A operand) 256..415 |
// S partial 416..479 | P (bf16 pairs, MMA A operand) 480..511.
// Shared memory: 4 x 40 KB KV stages | 32 KB landing buffer for the peer's partial S | 32 KB
// staging buffer for the outgoing partial.
//
// Warps (640 threads, registers redistributed with setmaxnreg): 0..9 = gather producers, 10 = MMA
// issuer (QK^T) / TMEM owner, 11 = MMA issuer (PV), 12..15 = senders (partial S: TMEM -> staging ->
// peer; Q -> TMEM), 16..19 = softmax + epilogue (thread = head = TMEM lane).  All waits are bounded; a wait that gives up sets the
// status word.
#pragma once

#include <stdlib.h>

#include "ptx_sm100.cuh"
#include "sfa_fwd_simt.cuh"

namespace dsa {

constexpr int kSfaHeads = 128;
// Tile size and ring depth (64 keys x 4 stages measured best: 48 keys x 5 stages, which also fits
// the 227 KB of shared memory, was 18 % slower - the cost of a tile is mostly fixed).
#ifndef DSA_SFA_BK
#define DSA_SFA_BK 64
#endif
#ifndef DSA_SFA_STAGES
#define DSA_SFA_STAGES 4
#endif
constexpr int kSfaBK = DSA_SFA_BK;      // keys per tile (a multiple of 16)
constexpr int kSfaStages = DSA_SFA_STAGES;
constexpr int kSfaHalf = kSfaBK / 2;   // the scores of a tile travel in two halves
static_assert(kSfaBK % 16 == 0 && kSfaBK <= 64 && kSfaHalf % 8 == 0, "tile size");
constexpr int kSfaThreads = 640;
constexpr int kSfaProducerWarps = 10;
constexpr int kSfaMmaWarp = 10;
constexpr int kSfaSendWarp0 = 12;    // warps 12..15: partial-score senders + Q loaders
constexpr int kSfaSoftWarp0 = 16;    // warps 16..19: softmax + epilogue
constexpr int kSfaDvHalf = 256;
constexpr int kSfaMaxSlots = 8192; // sparse_count * sparse_block_size served by this kernel

constexpr uint32_t kSfaBlk = kSfaBK * 128;                 // one 64-column block of a stage: BK rows x 128 B
constexpr uint32_t kSfaStage = 5 * kSfaBlk;                // (rank 1 uses 4 of the 5 blocks)
constexpr uint32_t kSfaOffX = kSfaStages * kSfaStage;
constexpr uint32_t kSfaXBytes = kSfaHeads * kSfaBK * 4;    // partial scores of a tile, fp32
constexpr uint32_t kSfaXHalfF = kSfaHeads * kSfaHalf;      // floats of one half (all heads)
constexpr uint32_t kSfaXWarpF = 32 * kSfaHalf;             // floats of one warp's part of a half
static_assert(kSfaStage % 1024 == 0, "stage alignment");
constexpr uint32_t kSfaOffStage = kSfaOffX + kSfaXBytes;  // outgoing copy of this CTA's partial S
constexpr uint32_t kSfaOffBar = kSfaOffStage + kSfaXBytes;
constexpr uint32_t kSfaSmemBytes = kSfaOffBar + 256;
static_assert(kSfaSmemBytes <= 232448, "shared memory");

constexpr uint32_t kTmO = 0, kTmQ = 256, kTmS = 416, kTmP = 480;
constexpr float kSfaRescaleTau = 8.f;  // log2 units: the running reference only moves when exceeded by this

struct SfaSm100Args {
  SfaDev p;
  int32_t* status;
  int32_t rows;
  uint32_t idesc_qk, idesc_pv;
  float scale_log2;  // scale * log2(e)
  int32_t is_bf16;
  long long* prof;   // optional: cycle counters of one thread per role (phase breakdown)
  const int2* nvalid;       // [rows * split] per work item: .x participating slots, .y first entry in key_list (pre-pass output)
  const int32_t* key_list;  // [rows, slots] their physical KV rows, front-packed
  // Split-KV (few query rows, e.g. decode at small batch): a row's slots are cut into `split` parts
  // of `part_keys` slots (a multiple of 64); work item v = row * split + part.  Each part leaves a
  // normalised fp32 partial output with its own maximum and sum, merged by sfa_merge_kernel.
  int32_t split, part_keys;
  int32_t items;            // rows * split
  float* part_o;            // [items, 128, 512] fp32 (split > 1)
  float* part_m;            // [items, 128] maximum of the scaled scores of the part (natural log units)
  float* part_l;            // [items, 128] sum of exp(score - maximum); 0 marks an empty part
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Pre-pass: one warp per query row.  Writes the physical KV rows of the slots that take part, in
// slot order, and their count.  A slot whose paged block is absent does not take part here.
__global__ void __launch_bounds__(128) sfa_compact_kernel(SfaDev p, int2* __restrict__ nvalid,
                                                          int32_t* __restrict__ key_list, int32_t split,
                                                          int32_t part_keys) {
  const int lane = threadIdx.x & 31;
  const int32_t row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const RowInfo ri = row_info(p.seq, row);
  const int32_t slots = p.sparse_count * p.sparse_block_size;
  const int32_t* idx_row = p.sparse_indices + (int64_t)row * p.sparse_count;
  int32_t* out = key_list + (int64_t)row * slots;
  int32_t n = 0;
  if (ri.pos < ri.act_q && ri.threshold > 0 && ri.act_k > 0) {
    for (int32_t j0 = 0; j0 < slots; j0 += 32) {
      const int32_t j = j0 + lane;
      int64_t prow = -1;
      if (j < slots) {
        const int32_t tok = sfa_slot_token(p, ri, idx_row, j);
        if (tok >= 0) prow = key_row(p.seq, ri, tok);
      }
      const uint32_t m = __ballot_sync(0xffffffffu, prow >= 0);
      if (prow >= 0) out[n + __popc(m & ((1u << lane) - 1u))] = (int32_t)prow;
      n += __popc(m);
    }
  }
  // the row's list is cut into `split` consecutive parts of `part_keys` entries
  if (lane < split)
    nvalid[(int64_t)row * split + lane] =
        make_int2(max(0, min(part_keys, n - lane * part_keys)), (int32_t)((int64_t)row * slots + lane * part_keys));
}

// kSplit: work items are parts of rows (split-KV) and leave fp32 partials; compiled apart so that the
// prefill instantiation carries none of it.
template <bool kSplit>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kSfaThreads, 1)
sfa_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_kn, const __grid_constant__ CUtensorMap tmap_kr,
                     const SfaSm100Args a) {
  extern __shared__ __align__(1024) unsigned char sfa_sm[];
  unsigned char* kv_s = sfa_sm;
  float* x_s = reinterpret_cast<float*>(sfa_sm + kSfaOffX);
  float* xo_s = reinterpret_cast<float*>(sfa_sm + kSfaOffStage);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sfa_sm + kSfaOffBar);
  uint64_t* kv_full = bars;                   // [stages] gather -> MMA
  uint64_t* kv_empty = bars + kSfaStages;     // [stages] MMA (PV done) -> gather
  uint64_t* q_full = bars + 2 * kSfaStages;   // softmax warps (Q stored in TMEM) -> MMA
  uint64_t* q_empty = q_full + 1;   // MMA (last QK of the token done) -> softmax warps
  uint64_t* s_full = q_full + 2;    // MMA -> softmax
  uint64_t* s_empty = q_full + 3;   // softmax (S in registers) -> MMA
  uint64_t* p_full = q_full + 4;    // softmax (P stored, O rescaled) -> MMA
  uint64_t* p_empty = q_full + 5;   // MMA (PV done) -> softmax
  uint64_t* o_free = q_full + 6;    // epilogue (O read out) -> MMA
  // The partial scores of a tile travel in two halves (keys 0..31 and 32..63), each with its own
  // 16 KB staging and landing buffer and its own barriers, so that the next tile's first half can be
  // on its way while the softmax warps still work on the current tile.
  uint64_t* x_full = q_full + 7;    // [2] peer's partial S has landed (transaction bytes)
  uint64_t* x_empty = q_full + 9;   // [2] peer has consumed what this CTA sent (remote arrivals)
  uint64_t* own_full = q_full + 11; // [2] senders: own partial is in the staging buffer -> softmax
  uint64_t* own_free = q_full + 13; // [2] softmax has read the staging buffer -> senders
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(q_full + 16);
  static_assert((2 * kSfaStages + 17) * 8 <= 256, "barrier area");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const uint32_t peer = rank ^ 1u;
  const int32_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int nblk = rank == 0 ? 5 : 4;          // 64-column blocks of this CTA's feature half
  const int nks = nblk * 4;                    // QK^T k-steps (16 dims each)

  const bool misaligned = (ptx::smem_u32(sfa_sm) & 1023u) != 0;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kSfaStages; ++i) { ptx::mbar_init(&kv_full[i], 1); ptx::mbar_init(&kv_empty[i], 1); }
    ptx::mbar_init(q_full, 128);
    ptx::mbar_init(q_empty, 1);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(s_empty, 128);
    ptx::mbar_init(p_full, 128);
    ptx::mbar_init(p_empty, 1);
    ptx::mbar_init(o_free, 128);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&x_full[i], 1);
      ptx::mbar_init(&x_empty[i], 4);
      ptx::mbar_init(&own_full[i], 4);
      ptx::mbar_init(&own_free[i], 4);
    }
    *abort_flag = misaligned ? 1 : 0;
    ptx::mbar_fence_init();
  }
  if (warp == kSfaMmaWarp) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // the peer's barriers must exist before anything is sent to it
  ptx::cluster_arrive();
  ptx::cluster_wait();
  const uint32_t tmem = *tmem_slot;
  // 512 threads start with 128 registers each; every role branch below first trades registers:
  // the softmax warps need more, everyone else less (whole warpgroups of 4 warps change together).

  const int32_t n1 = a.p.n1;                   // real heads (<= 128); lanes past them carry zero queries
  const int32_t n1d = n1 * a.p.d;

  if (warp < kSfaSendWarp0) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
   if (*abort_flag) {
    // nothing started: fall through to the teardown
  } else if (warp < kSfaProducerWarps) {
    // ------------------------------------------------------------------ gather producers
    // A tile is 16 row groups (4 keys each) x nblk column blocks = 80 (rank 0) or 64 (rank 1)
    // gather4 loads of 512 bytes.  A warp issues one such load every ~67 cycles whatever the lane
    // pattern, but warps issue in parallel, so the loads of every tile are dealt out over ten
    // warps (load o goes to warp o % 10, lane o / 10).  Warp 0 also arms the stage's barrier.
    uint32_t n_tile = 0;
    bool ok = true;
    long long pprof[4] = {0, 0, 0, 0};
    const int nops = (kSfaBK / 4) * nblk;
    const int o = warp + kSfaProducerWarps * lane;     // this lane's load of every tile
    const int grp = o / nblk, blk = o - grp * nblk;     // row group, column block
    const bool active = o < nops;
    const int32_t x = rank == 0 ? (blk < 4 ? blk * 64 : 0) : kSfaDvHalf + blk * 64;
    const CUtensorMap* tm = (rank == 0 && blk == 4) ? &tmap_kr : &tmap_kn;
    if (lane == 0) { ptx::prefetch_tmap(&tmap_kn); ptx::prefetch_tmap(&tmap_kr); }
    // The row numbers of a tile come from global memory (the pre-pass list); they are fetched one
    // tile ahead so that their latency never sits between a freed stage and the gather.
    struct TilePos { int32_t row, t, ntiles, nvalid, off; };
    auto first_from = [&](int32_t row) -> TilePos {   // `row` counts work items here
      for (; row < a.items; row += n_clusters) {
        const int2 d = a.nvalid[row];
        if (d.x > 0) return TilePos{row, 0, (d.x + kSfaBK - 1) / kSfaBK, d.x, d.y};
      }
      return TilePos{a.items, 0, 0, 0, 0};
    };
    auto load_rows = [&](const TilePos& tp, int32_t* r) {
      const int32_t* list = a.key_list + tp.off;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int32_t k = tp.t * kSfaBK + grp * 4 + i;
        // keys past the end of the row re-read the tile's first key
        r[i] = (active && tp.row < a.items) ? list[k < tp.nvalid ? k : tp.t * kSfaBK] : 0;
      }
    };
    TilePos cur = first_from(cluster_id);
    int32_t rc[4], rn[4];
    load_rows(cur, rc);
    while (cur.row < a.items && ok) {
      TilePos nxt = cur;
      if (++nxt.t >= nxt.ntiles) nxt = first_from(cur.row + n_clusters);
      load_rows(nxt, rn);
      const uint32_t s = n_tile % kSfaStages, use = n_tile / kSfaStages;
      const long long p1 = clock64();
      if (lane == 0) ok = ptx::mbar_wait(&kv_empty[s], (use & 1) ^ 1, abort_flag);
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      if (!ok) break;
      const long long p2 = clock64();
      if (warp == 0 && lane == 0) ptx::mbar_arrive_expect_tx(&kv_full[s], kSfaBK * nblk * 128);
      if (active)
        ptx::tma_gather4_2d(kv_s + s * kSfaStage + blk * kSfaBlk + grp * 512, tm, &kv_full[s], x, rc[0], rc[1], rc[2],
                            rc[3]);
      __syncwarp();
      pprof[1] += p2 - p1; pprof[2] += clock64() - p2;
      ++n_tile;
      cur = nxt;
#pragma unroll
      for (int i = 0; i < 4; ++i) rc[i] = rn[i];
    }
    if (a.prof != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
      for (int i = 0; i < 4; ++i) a.prof[16 + i] = pprof[i];
    }
  } else if (warp == kSfaMmaWarp) {
    // ------------------------------------------------------------------ QK^T issuer (warp 6)
    // S = Q_c K_c^T for every tile, as early as the KV ring and the single S buffer allow; it
    // never waits for the softmax, so the score exchange of later tiles overlaps the softmax of
    // earlier ones.
    uint32_t n_tile = 0, n_tok = 0;
    bool ok = true;
    long long mprof[4] = {0, 0, 0, 0};
    const uint32_t kv_addr = ptx::smem_u32(kv_s);
    for (int32_t row = cluster_id; row < a.items && ok; row += n_clusters) {   // work items
      const int32_t nvalid = a.nvalid[row].x;
      const int32_t ntiles = (nvalid + kSfaBK - 1) / kSfaBK;
      if (ntiles == 0) continue;
      if (lane == 0) {
        ok = ptx::mbar_wait(q_full, n_tok & 1, abort_flag);
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          const uint32_t s = n_tile % kSfaStages, use = n_tile / kSfaStages;
          const long long m0 = clock64();
          ok = ptx::mbar_wait(&kv_full[s], use & 1, abort_flag);
          if (!ok) break;
          const long long m1 = clock64();
          ok = ptx::mbar_wait(s_empty, (n_tile & 1) ^ 1, abort_flag);
          if (!ok) break;
          mprof[0] += m1 - m0; mprof[1] += clock64() - m1;
          ptx::tc_fence_after();
          for (int ks = 0; ks < nks; ++ks) {
            const uint64_t bd = ptx::desc_kmajor_sw128(kv_addr + s * kSfaStage + (ks >> 2) * kSfaBlk + (ks & 3) * 32);
            ptx::mma_ts(tmem + kTmS, tmem + kTmQ + ks * 8, bd, a.idesc_qk, ks > 0 ? 1u : 0u);
          }
          ptx::mma_commit(s_full);
          if (t == ntiles - 1) ptx::mma_commit(q_empty);
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      n_tile = __shfl_sync(0xffffffffu, n_tile, 0);
      ++n_tok;
    }
    if (a.prof != nullptr && blockIdx.x == 0 && lane == 0) {
      for (int i = 0; i < 2; ++i) a.prof[12 + i] = mprof[i];
    }
  } else if (warp == kSfaMmaWarp + 1) {
    // ------------------------------------------------------------------ PV issuer (warp 7)
    // O (+)= P V_c once the softmax warps have stored P; frees the KV stage and the P buffer.
    uint32_t n_tile = 0, n_tok = 0;
    bool ok = true;
    long long wait_p = 0;
    const uint32_t kv_addr = ptx::smem_u32(kv_s);
    for (int32_t row = cluster_id; row < a.items && ok; row += n_clusters) {   // work items
      const int32_t nvalid = a.nvalid[row].x;
      const int32_t ntiles = (nvalid + kSfaBK - 1) / kSfaBK;
      if (ntiles == 0) continue;
      if (lane == 0) {
        ok = ptx::mbar_wait(o_free, (n_tok & 1) ^ 1, abort_flag);   // previous token's O has been read out
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          const uint32_t s = n_tile % kSfaStages, use = n_tile / kSfaStages;
          ok = ptx::mbar_wait(&kv_full[s], use & 1, abort_flag);    // long complete; observed for ordering
          if (!ok) break;
          const long long m0 = clock64();
          ok = ptx::mbar_wait(p_full, n_tile & 1, abort_flag);
          if (!ok) break;
          wait_p += clock64() - m0;
          ptx::tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < kSfaBK / 16; ++ks) {
            const uint64_t bd = ptx::desc_mnmajor_sw128(kv_addr + s * kSfaStage + ks * 16 * 128, kSfaBlk, 1024);
            ptx::mma_ts(tmem + kTmO, tmem + kTmP + ks * 8, bd, a.idesc_pv, (t == 0 && ks == 0) ? 0u : 1u);
          }
          ptx::mma_commit(p_empty);
          ptx::mma_commit(&kv_empty[s]);
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      n_tile = __shfl_sync(0xffffffffu, n_tile, 0);
      ++n_tok;
    }
    if (a.prof != nullptr && blockIdx.x == 0 && lane == 0) a.prof[14] = wait_p;
  }
  } else if (warp < kSfaSoftWarp0) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    if (!*abort_flag) {
    // ------------------------------------------------------------------ senders
    // Per token: this CTA's Q half into tensor memory.  Per tile: the partial S from tensor memory
    // into the staging buffer (warp w owns 8 KB: 16-byte chunk c of a lane at w * 8192 + c * 512 +
    // lane * 16), one bulk copy per warp into the peer's landing buffer (counted on the peer's
    // x_full barrier), and a local hand-over of the same staging buffer to the softmax warps.
    const int quarter = warp & 3;
    const int h = quarter * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t x_peer = ptx::map_to_rank(x_s, peer);
    const uint32_t x_full_peer = ptx::map_to_rank(x_full, peer);
    uint32_t n_tile = 0, n_tok = 0;
    bool ok = true;
    long long sprof[4] = {0, 0, 0, 0};
    auto wait_w = [&](uint64_t* bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag));
    };
    auto wait_wc = [&](uint64_t* bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, ptx::mbar_wait_cluster(bar, parity, abort_flag));
    };
    auto q_half = [&](int32_t r) -> const uint4* {
      return reinterpret_cast<const uint4*>((const unsigned char*)a.p.query +
                                            ((int64_t)r * n1d + (int64_t)h * a.p.d + rank * kSfaDvHalf) * 2);
    };
    auto q_rope = [&](int32_t r) -> const uint4* {
      return reinterpret_cast<const uint4*>((const unsigned char*)a.p.query_rope +
                                            ((int64_t)r * n1 + h) * a.p.d_rope * 2);
    };
    for (int32_t item = cluster_id; item < a.items && ok; item += n_clusters) {
      const int32_t nvalid = a.nvalid[item].x;
      const int32_t ntiles = (nvalid + kSfaBK - 1) / kSfaBK;
      if (ntiles == 0) continue;
      const int32_t row = kSplit ? item / a.split : item;   // the query row of this work item
      // ---- this token's Q half -> tensor memory (bf16 pairs, row h in lane h)
      ok = wait_w(q_empty, (n_tok & 1) ^ 1);
      if (!ok) break;
      ptx::tc_fence_after();
      {
        // 16 loads in flight per batch (a batch of 8 left the five batches' latencies in a row at
        // every token boundary)
        const uint4* qn = q_half(row);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t w[64];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint4 v = h < n1 ? __ldg(qn + c * 16 + i) : make_uint4(0, 0, 0, 0);
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
          }
          ptx::tmem_st_x32(lane_addr + kTmQ + c * 64, w);
          ptx::tmem_st_x32(lane_addr + kTmQ + c * 64 + 32, w + 32);
        }
        if (rank == 0) {
          const uint4* qr = q_rope(row);
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint4 v = h < n1 ? __ldg(qr + i) : make_uint4(0, 0, 0, 0);
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
          }
          ptx::tmem_st_x32(lane_addr + kTmQ + 128, w);
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        ptx::mbar_arrive(q_full);
        // the next token's Q rows go to L2 now, a whole token's worth of tiles before they are read
        int32_t nitem = item + n_clusters;
        while (nitem < a.items && a.nvalid[nitem].x == 0) nitem += n_clusters;
        if (nitem < a.items && h < n1) {
          const int32_t nrow = kSplit ? nitem / a.split : nitem;
          const unsigned char* nq = reinterpret_cast<const unsigned char*>(q_half(nrow));
#pragma unroll
          for (int i = 0; i < 4; ++i) ptx::prefetch_l2(nq + i * 128);
          if (rank == 0) ptx::prefetch_l2(q_rope(nrow));
        }
      }
      for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
        const long long s0 = clock64();
        ok = wait_w(s_full, n_tile & 1);
        if (!ok) break;
        sprof[0] += clock64() - s0;
        ptx::tc_fence_after();
        float sv[64];   // kSfaBK of them are scores
        ptx::tmem_ld_x32(lane_addr + kTmS, reinterpret_cast<uint32_t*>(sv));
        if (kSfaBK > 48) ptx::tmem_ld_x32(lane_addr + kTmS + 32, reinterpret_cast<uint32_t*>(sv) + 32);
        else if (kSfaBK > 32) ptx::tmem_ld_x16(lane_addr + kTmS + 32, reinterpret_cast<uint32_t*>(sv) + 32);
        ptx::tmem_ld_wait();
        ptx::tc_fence_before();
        ptx::mbar_arrive(s_empty);
        // a staging half is free once the peer has consumed what was copied out of it and the
        // local softmax warps have read it (half hf: kSfaXWarpF floats per warp, 16-byte chunk c of
        // a lane at c * 512 + lane * 16 inside the warp's part)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const long long s1 = clock64();
          ok = wait_wc(&x_empty[hf], (n_tile & 1) ^ 1);
          if (!ok) break;
          const long long s2 = clock64();
          ok = wait_w(&own_free[hf], (n_tile & 1) ^ 1);
          if (!ok) break;
          sprof[1] += s2 - s1; sprof[2] += clock64() - s2;
          if (quarter == 0 && lane == 0) ptx::mbar_arrive_expect_tx(&x_full[hf], kSfaXBytes / 2);  // arm my landing half
          float* mine = xo_s + hf * kSfaXHalfF + quarter * kSfaXWarpF + lane * 4;
#pragma unroll
          for (int c = 0; c < kSfaBK / 8; ++c) {
            const int k = hf * kSfaHalf + 4 * c;
            *reinterpret_cast<float4*>(mine + c * 128) = make_float4(sv[k], sv[k + 1], sv[k + 2], sv[k + 3]);
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            ptx::bulk_copy_to_peer(x_peer + (hf * kSfaXHalfF + quarter * kSfaXWarpF) * 4,
                                   xo_s + hf * kSfaXHalfF + quarter * kSfaXWarpF, kSfaXWarpF * 4, x_full_peer + hf * 8);
            ptx::mbar_arrive(&own_full[hf]);
          }
        }
      }
      ++n_tok;
    }
    if (a.prof != nullptr && blockIdx.x == 0 && quarter == 0 && lane == 0) {
      for (int i = 0; i < 3; ++i) a.prof[20 + i] = sprof[i];
    }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    if (!*abort_flag) {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quarter = warp & 3;
    const int h = quarter * 32 + lane;                       // head == TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t x_empty_peer = ptx::map_to_rank(x_empty, peer);
    uint32_t n_tile = 0;
    bool ok = true;
    long long prof[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};  // cycle sums per phase (stored only when profiling)
    // waits of these warps are made warp-uniform: the tcgen05 loads / stores that follow are
    // warp-collective and must never run with part of a warp gone
    auto wait_w = [&](uint64_t* bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag));
    };
    auto wait_wc = [&](uint64_t* bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, ptx::mbar_wait_cluster(bar, parity, abort_flag));
    };
    for (int32_t item = cluster_id; item < a.items && ok; item += n_clusters) {
      const int32_t nvalid = a.nvalid[item].x;
      const int32_t ntiles = (nvalid + kSfaBK - 1) / kSfaBK;
      const int32_t row = kSplit ? item / a.split : item;
      unsigned char* out_row = (unsigned char*)a.p.out + ((int64_t)row * n1d + (int64_t)h * a.p.d + rank * kSfaDvHalf) * 2;
      float* part_row = kSplit ? a.part_o + ((int64_t)item * kSfaHeads + h) * (2 * kSfaDvHalf) + rank * kSfaDvHalf
                                    : nullptr;
      if (ntiles == 0) {
        if constexpr (kSplit) {
          // an empty part: the merge skips it
          if (rank == 0) { a.part_m[(int64_t)item * kSfaHeads + h] = 0.f; a.part_l[(int64_t)item * kSfaHeads + h] = 0.f; }
        } else {
          // nothing visible: zeros in all three outputs
          if (h < n1) {
#pragma unroll
            for (int c = 0; c < kSfaDvHalf * 2 / 16; ++c) reinterpret_cast<uint4*>(out_row)[c] = make_uint4(0, 0, 0, 0);
            if (rank == 0 && a.p.return_lse) {
              a.p.softmax_max[(int64_t)row * n1 + h] = 0.f;
              a.p.softmax_sum[(int64_t)row * n1 + h] = 0.f;
            }
          }
        }
        continue;
      }
      float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
      for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
        const long long c0 = clock64();
        const int32_t cnt = min(kSfaBK, nvalid - t * kSfaBK);
        // ---- full S = own partial (staging halves) + the peer's partial (landing halves); each
        // half is handed back as soon as it has been read
        float sc[kSfaBK];
        long long c1 = c0;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          ok = wait_wc(&x_full[hf], n_tile & 1);
          if (!ok) break;
          ok = wait_w(&own_full[hf], n_tile & 1);
          if (!ok) break;
          if (hf == 0) c1 = clock64();
          const float* theirs = x_s + hf * kSfaXHalfF + quarter * kSfaXWarpF + lane * 4;
          const float* mine = xo_s + hf * kSfaXHalfF + quarter * kSfaXWarpF + lane * 4;
          float dep = 0.f;
#pragma unroll
          for (int c = 0; c < kSfaBK / 8; ++c) {
            const float4 v = *reinterpret_cast<const float4*>(theirs + c * 128);
            const float4 o = *reinterpret_cast<const float4*>(mine + c * 128);
            const int k = hf * kSfaHalf + 4 * c;
            sc[k] = v.x + o.x; sc[k + 1] = v.y + o.y; sc[k + 2] = v.z + o.z; sc[k + 3] = v.w + o.w;
            dep += sc[k] + sc[k + 1] + sc[k + 2] + sc[k + 3];
          }
          __syncwarp();
          if (lane == 0) {
            // relaxed: nothing is published, the peer only learns that the reads are done (`dep`
            // depends on every load of this half)
            ptx::mbar_arrive_remote_relaxed(x_empty_peer + hf * 8, __float_as_uint(dep));
            ptx::mbar_arrive(&own_free[hf]);
          }
        }
        if (!ok) break;
        // ---- softmax in the log2 domain; keys past `cnt` are padding
        if (cnt == kSfaBK) {
#pragma unroll
          for (int k = 0; k < kSfaBK; ++k) sc[k] *= a.scale_log2;
        } else {
#pragma unroll
          for (int k = 0; k < kSfaBK; ++k) sc[k] = k < cnt ? sc[k] * a.scale_log2 : -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int k = 0; k < kSfaBK; k += 4) {
          mx4[0] = fmaxf(mx4[0], sc[k]); mx4[1] = fmaxf(mx4[1], sc[k + 1]);
          mx4[2] = fmaxf(mx4[2], sc[k + 2]); mx4[3] = fmaxf(mx4[3], sc[k + 3]);
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const long long c2 = clock64();
        m_true = fmaxf(m_true, mx);
        float alpha = 1.f;
        bool rescale = false;
        if (t == 0) {
          m_ref = mx;
        } else if (mx > m_ref + kSfaRescaleTau) {
          alpha = ex2(m_ref - mx);
          m_ref = mx;
          rescale = true;
        }
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < kSfaBK; k += 4) {
          sc[k] = ex2(sc[k] - m_ref); sc[k + 1] = ex2(sc[k + 1] - m_ref);
          sc[k + 2] = ex2(sc[k + 2] - m_ref); sc[k + 3] = ex2(sc[k + 3] - m_ref);
          sum4[0] += sc[k]; sum4[1] += sc[k + 1]; sum4[2] += sc[k + 2]; sum4[3] += sc[k + 3];
        }
        l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        if (ntiles == 1) {
          // a single tile holds the whole row: normalise before rounding, as the golden does
          const float inv = 1.f / l;
#pragma unroll
          for (int k = 0; k < kSfaBK; ++k) sc[k] *= inv;
        }
        const long long c3 = clock64();
        // ---- P (and, rarely, a rescaled O) -> tensor memory once the previous PV has finished
        ok = wait_w(p_empty, (n_tile & 1) ^ 1);
        const long long c4 = clock64();
        if (!ok) break;
        ptx::tc_fence_after();
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int c = 0; c < kSfaDvHalf / 32; ++c) {
            uint32_t o[32];
            ptx::tmem_ld_x32(lane_addr + kTmO + c * 32, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            ptx::tmem_st_x32(lane_addr + kTmO + c * 32, o);
          }
        }
        {
          uint32_t pw[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) pw[i] = i < kSfaBK / 2 ? pack2(sc[2 * i], sc[2 * i + 1], a.is_bf16) : 0u;
          ptx::tmem_st_x32(lane_addr + kTmP, pw);
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        ptx::mbar_arrive(p_full);
        prof[0] += c1 - c0; prof[1] += c2 - c1; prof[2] += c3 - c2; prof[3] += c4 - c3; prof[4] += clock64() - c4;
        prof[5] += 1;
      }
      if (!ok) break;
      // ---- epilogue: wait for the last PV, normalise, store
      const long long ce0 = clock64();
      ok = wait_w(p_empty, (n_tile & 1) ^ 1);
      if (!ok) break;
      prof[8] += clock64() - ce0;
      ptx::tc_fence_after();
      const float inv = ntiles == 1 ? 1.f : 1.f / l;
#pragma unroll 1
      for (int c = 0; c < kSfaDvHalf / 32; ++c) {
        uint32_t o[32];
        ptx::tmem_ld_x32(lane_addr + kTmO + c * 32, o);
        ptx::tmem_ld_wait();
        if constexpr (kSplit) {
          // split-KV: the normalised partial output stays fp32 for the merge
#pragma unroll
          for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(part_row + c * 32)[i] =
                make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                            __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
        } else {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            w[i] = pack2(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv, a.is_bf16);
          // whole 32-byte sectors per store: a lane's row is 1 KB away from its neighbour's, so every
          // store of a warp touches 32 different lines and the request count is what costs
          if (h < n1) {
            ptx::st_global_v8(out_row + c * 64, w);
            ptx::st_global_v8(out_row + c * 64 + 32, w + 8);
          }
        }
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(o_free);
      prof[7] += clock64() - ce0;
      if constexpr (kSplit) {
        if (rank == 0) {
          a.part_m[(int64_t)item * kSfaHeads + h] = m_true * 0.6931471805599453f;
          a.part_l[(int64_t)item * kSfaHeads + h] = l * ex2(m_ref - m_true);
        }
      } else if (rank == 0 && a.p.return_lse && h < n1) {
        // max of the scaled scores and sum of exp(score - max), back from the log2 domain
        a.p.softmax_max[(int64_t)row * n1 + h] = m_true * 0.6931471805599453f;
        a.p.softmax_sum[(int64_t)row * n1 + h] = l * ex2(m_ref - m_true);
      }
    }
    if (a.prof != nullptr && blockIdx.x == 0 && quarter == 0 && lane == 0) {
#pragma unroll
      for (int i = 0; i < 12; ++i) a.prof[i] = prof[i];
    }
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies / MMAs in flight land
  }
  ptx::tc_fence_before();
  __syncthreads();
  // neither CTA may leave while its peer can still write into its shared memory
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == kSfaMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(a.status, misaligned ? 2 : 1);
}

// ---- host side ---------------------------------------------------------------------------------
inline bool sfa_sm100_eligible(const DsaSfaParams* p) {
  // fewer than 128 heads (a tensor-parallel shard) run with the spare lanes carrying zero queries;
  // below 16 heads the portable kernel wastes less
  if (p->n1 < 16 || p->n1 > kSfaHeads || p->d != 512 || p->d_rope != 64) return false;
  if ((int64_t)p->sparse_count * p->sparse_block_size > kSfaMaxSlots) return false;
  if (((uintptr_t)p->query & 15u) || ((uintptr_t)p->query_rope & 15u) || ((uintptr_t)p->key & 15u) ||
      ((uintptr_t)p->key_rope & 15u) || ((uintptr_t)p->out & 31u))
    return false;
  if (p->key_rows < 1 || p->key_rows >= (1ll << 31)) return false;
  const int64_t rows_ = p->layout_q == DSA_LAYOUT_TND ? p->s1 : (int64_t)p->batch * p->s1;
  if (rows_ * p->sparse_count * p->sparse_block_size >= (1ll << 31)) return false;   // key_list offsets are int32
  return true;
}

// Merge of the split-KV partials: one CTA per query row and group of 8 heads, thread = 4 output
// columns of one head at a time.  out = sum_p w_p O_p / sum_p w_p with w_p = l_p exp(m_p - max_p m_p); empty parts have l = 0.
__global__ void __launch_bounds__(256) sfa_merge_kernel(SfaDev p, int32_t split, const float* __restrict__ part_o,
                                                        const float* __restrict__ part_m,
                                                        const float* __restrict__ part_l, int32_t is_bf16) {
  const int32_t row = blockIdx.x;
  // blockIdx.y: group of 8 heads
  for (int32_t e = threadIdx.x; e < 8 * (2 * kSfaDvHalf / 4); e += 256) {
    const int32_t h = blockIdx.y * 8 + e / (2 * kSfaDvHalf / 4), c4 = e % (2 * kSfaDvHalf / 4);
    if (h >= p.n1) continue;
    float mx = -INFINITY;
    for (int32_t q = 0; q < split; ++q) {
      const int64_t i = ((int64_t)row * split + q) * kSfaHeads + h;
      if (part_l[i] > 0.f) mx = fmaxf(mx, part_m[i]);
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
    for (int32_t q = 0; q < split; ++q) {
      const int64_t i = ((int64_t)row * split + q) * kSfaHeads + h;
      const float l = part_l[i];
      if (l > 0.f) {
        const float w = l * __expf(part_m[i] - mx);
        const float4 o = reinterpret_cast<const float4*>(part_o + i * (2 * kSfaDvHalf))[c4];
        acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
        den += w;
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    uint2 packed;
    packed.x = pack2(acc.x * inv, acc.y * inv, is_bf16);
    packed.y = pack2(acc.z * inv, acc.w * inv, is_bf16);
    reinterpret_cast<uint2*>((unsigned char*)p.out + ((int64_t)row * p.n1 + h) * (2 * kSfaDvHalf) * 2)[c4] = packed;
    if (c4 == 0 && p.return_lse) {
      p.softmax_max[(int64_t)row * p.n1 + h] = den > 0.f ? mx : 0.f;
      p.softmax_sum[(int64_t)row * p.n1 + h] = den;
    }
  }
}

// Split factor: only when there are too few query rows to give every CTA pair one (decode at small
// batch); at least four 64-key tiles per part.  74 CTA pairs are assumed here (the answer must not
// depend on the device, the workspace size is derived from it); any other count is still correct.
inline int32_t sfa_sm100_split(int64_t rows, int64_t slots) {
  const int64_t pairs = 74;
  if (rows < 1 || rows * 2 > pairs) return 1;
  int64_t s = pairs / rows;
  const int64_t tiles = (slots + kSfaBK - 1) / kSfaBK;
  if (s > tiles / 4) s = tiles / 4;
  if (s > 8) s = 8;
  return s < 2 ? 1 : (int32_t)s;
}
inline int32_t sfa_sm100_part_keys(int64_t slots, int32_t split) {
  const int64_t tiles = (slots + kSfaBK - 1) / kSfaBK;
  return (int32_t)(((tiles + split - 1) / split) * kSfaBK);
}

// Workspace beyond the header: nvalid[rows * split], key_list[rows * slots], and for split > 1 the
// partial maxima, sums and outputs.
struct SfaWsLayout { size_t nvalid, key_list, part_m, part_l, part_o, total; };
inline SfaWsLayout sfa_sm100_ws_layout(int64_t rows, int64_t slots) {
  const int32_t split = sfa_sm100_split(rows, slots);
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  SfaWsLayout w;
  w.nvalid = 0;
  w.key_list = up((size_t)rows * split * 8);
  w.part_m = w.key_list + up((size_t)rows * slots * 4);
  const size_t stats = split > 1 ? up((size_t)rows * split * kSfaHeads * 4) : 0;
  w.part_l = w.part_m + stats;
  w.part_o = w.part_l + stats;
  w.total = w.part_o + (split > 1 ? (size_t)rows * split * kSfaHeads * 2 * kSfaDvHalf * 4 : 0);
  return w;
}
inline size_t sfa_sm100_workspace_bytes(const DsaSfaParams* p) {
  const int64_t rows = p->layout_q == DSA_LAYOUT_TND ? p->s1 : (int64_t)p->batch * p->s1;
  const int64_t slots = (int64_t)p->sparse_count * p->sparse_block_size;
  return sfa_sm100_ws_layout(rows, slots).total;
}

inline int sfa_sm100_launch(const DsaSfaParams* p, const SfaDev& d, int32_t* status, void* scratch, cudaStream_t st) {
  static int sm_count[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DSA_ERR_CUDA;
  if (sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 2) return DSA_ERR_CUDA;
    if (cudaFuncSetAttribute(sfa_fwd_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSfaSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(sfa_fwd_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSfaSmemBytes) != cudaSuccess)
      return DSA_ERR_CUDA;
    sm_count[dev] = n;
  }
  const bool bf16 = p->dtype == DSA_DTYPE_BF16;
  const int64_t slots = (int64_t)p->sparse_count * p->sparse_block_size;
  const SfaWsLayout w = sfa_sm100_ws_layout(d.rows, slots);
  const int32_t split = sfa_sm100_split(d.rows, slots);
  const int32_t part_keys = split > 1 ? sfa_sm100_part_keys(slots, split) : (int32_t)((slots + kSfaBK - 1) / kSfaBK) * kSfaBK;
  int2* nvalid = reinterpret_cast<int2*>((char*)scratch + w.nvalid);
  int32_t* key_list = reinterpret_cast<int32_t*>((char*)scratch + w.key_list);
  sfa_compact_kernel<<<(d.rows + 3) / 4, 128, 0, st>>>(d, nvalid, key_list, split, part_keys);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  SfaSm100Args a;
  a.p = d;
  a.status = status;
  a.rows = d.rows;
  a.idesc_qk = ptx::idesc_f16(bf16 ? 1u : 0u, 128, kSfaBK, 0, 0);
  a.idesc_pv = ptx::idesc_f16(bf16 ? 1u : 0u, 128, kSfaDvHalf, 0, 1);
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.is_bf16 = bf16 ? 1 : 0;
  a.prof = getenv("DSA_SFA_PROFILE") ? reinterpret_cast<long long*>(status + 16) : nullptr;
  a.nvalid = nvalid;
  a.key_list = key_list;
  a.split = split;
  a.part_keys = part_keys;
  a.items = d.rows * split;
  a.part_m = reinterpret_cast<float*>((char*)scratch + w.part_m);
  a.part_l = reinterpret_cast<float*>((char*)scratch + w.part_l);
  a.part_o = reinterpret_cast<float*>((char*)scratch + w.part_o);
  int clusters = sm_count[dev] / 2;
  if (clusters > a.items) clusters = a.items;
  CUtensorMap tkn, tkr;
  if (!make_tmap_gather4_16bit(&tkn, p->key, (uint64_t)p->key_rows, 512, 1024, 64, bf16)) return DSA_ERR_CUDA;
  if (!make_tmap_gather4_16bit(&tkr, p->key_rope, (uint64_t)p->key_rows, 64, 128, 64, bf16)) return DSA_ERR_CUDA;
  if (split > 1) sfa_fwd_sm100_kernel<true><<<clusters * 2, kSfaThreads, kSfaSmemBytes, st>>>(tkn, tkr, a);
  else sfa_fwd_sm100_kernel<false><<<clusters * 2, kSfaThreads, kSfaSmemBytes, st>>>(tkn, tkr, a);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  if (split > 1) {
    sfa_merge_kernel<<<dim3(d.rows, kSfaHeads / 8), 256, 0, st>>>(d, split, a.part_o, a.part_m, a.part_l, a.is_bf16);
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  }
  return DSA_OK;
}

}  // namespace dsa
