// Sparse flash attention forward on tcgen05 tensor cores for the MLA-absorb production shape:
// up to 128 query heads, D = 512 (+64 rope), one KV head, any layout, token- or block-wise
// indices.  16..127 heads (a tensor-parallel shard of the 128) run the same code with the spare
// accumulator rows carrying zero queries; few query rows (decode at small batch) are split along
// their keys into parts whose partial results a small kernel merges.
//
// One query token is processed by a CTA PAIR (a 2-CTA cluster) that splits the HEADS: CTA c owns
// heads 64c..64c+63, i.e. its own rows of S = Q K^T and of O = P V, so the softmax of a row never
// needs data from the other CTA.  Both contractions are pair MMAs (tcgen05.mma.cta_group::2,
// M = 128 = 2 x 64 rows): each CTA feeds its own A rows and HALF of the B operand, which the
// hardware shares between the two tensor cores.  That fixes what each CTA has to gather:
//   S tile  [128 heads x 64 keys]  : B = K rows, split along the keys  -> CTA c gathers 32 of the
//                                    tile's 64 keys with all 576 features  (36 KB, K-major)
//   O       [128 heads x 512 cols] : B = V rows, split along the value columns -> CTA c gathers
//                                    all 64 keys, columns {c*128.., 256+c*128..} (32 KB, MN-major)
// (two N = 256 MMAs per 16-key step: the first produces value columns 0..255, the second
// 256..511).  The two operand blocks of a CTA cannot alias: a pair MMA reads both CTAs at the SAME
// shared-memory offsets, the score product needs identical features at an offset and the value
// product identical keys.  Gathers are TMA tile::gather4 loads into the 128-byte-swizzled MMA
// layout, issued by twelve producer warps from a front-packed list of physical KV rows that a
// pre-pass kernel writes.
//
// Accumulator layout of a pair MMA with M = 128 (measured): lanes 0..63 hold a CTA's rows with the
// first half of N, lanes 64..127 the same rows with the second half.  So TMEM lane L of CTA c
// belongs to head 64c + (L & 63); for S it holds the tile's keys 32*(L>>6) .. +31, for O the value
// columns j*256 + 128*(L>>6) .. +127 of MMA j.  The two threads of a head exchange their running
// maxima and sums through shared memory.
//
// Tensor memory per CTA: O 0..255 | S (two buffers) 256..319.
// Shared memory per CTA: Q_c 72 KB (A operand, loaded per token by TMA) | 2 x 36 KB K slots |
// 2 x 32 KB V slots | 2 x 8 KB P (A operand of the value product, written by the softmax warps).
//
// Warps (640 threads): 0..5 K producers, 6..11 V producers, 12/13 QK^T issuers (even / odd tiles,
// two issuing threads keep the tensor pipe fed with the short N = 64 MMAs), 14 PV issuer, 15 Q
// loader, 16..19 softmax + epilogue.  MMAs are issued by the even CTA only; in the odd CTA the
// issuer warps relay "my operand has landed" to the even CTA's barriers instead.  All waits are
// bounded; a wait that gives up sets the status word.
#pragma once

#include <atomic>
#include <mutex>

#include "ptx_sm100.cuh"
#include "sfa_fwd_simt.cuh"

namespace dsa {

constexpr int kSfaHeads = 128;       // heads per CTA pair
constexpr int kSfaCtaHeads = 64;
constexpr int kSfaBK = 64;           // keys per tile
constexpr int kSfaHalfBK = 32;       // keys of a tile each CTA gathers for the score product
constexpr int kSfaThreads = 768;
constexpr int kSfaQkLanes = 3;       // QK^T issuers; issuer i owns feature blocks 3i..3i+2 and a partial S
constexpr int kSfaKWarps = 9;        // warps 0..8: K gather producers, three per issuer
constexpr int kSfaQWarp = 9;         // Q loader (warps 10, 11 idle)
constexpr int kSfaQkWarp0 = 12;      // warps 12..14
constexpr int kSfaPvWarp = 15;
constexpr int kSfaCopyWarp0 = 16;    // warps 16..19: V copiers
constexpr int kSfaSoftWarp0 = 20;    // warps 20..23
constexpr int kSfaDv = 512;
constexpr int kSfaMaxSlots = 8192;   // sparse_count * sparse_block_size served by this kernel

constexpr uint32_t kSfaQBlk = kSfaCtaHeads * 128;            // 64 heads x 64 features
constexpr uint32_t kSfaQBytes = 9 * kSfaQBlk;                // 73 728
constexpr uint32_t kSfaKBlk = kSfaHalfBK * 128;              // 32 keys x 64 features
constexpr uint32_t kSfaKSlot = 9 * kSfaKBlk;                 // 36 864
constexpr uint32_t kSfaKSub = 3 * kSfaKBlk;                  // the three blocks of one issuer
constexpr uint32_t kSfaVBlk = kSfaBK * 128;                  // 64 keys x 64 value columns
constexpr uint32_t kSfaVSlot = 4 * kSfaVBlk;                 // 32 768
constexpr uint32_t kSfaPBuf = kSfaCtaHeads * kSfaBK * 2;     // 8 192
constexpr uint32_t kSfaOffQ = 0;
constexpr uint32_t kSfaOffK = kSfaOffQ + kSfaQBytes;
constexpr uint32_t kSfaOffV = kSfaOffK + 2 * kSfaKSlot;
constexpr uint32_t kSfaOffP = kSfaOffV + 2 * kSfaVSlot;
constexpr uint32_t kSfaOffX = kSfaOffP + 2 * kSfaPBuf;       // float xm[2][128], xs[128]
constexpr uint32_t kSfaOffBar = kSfaOffX + 3 * 128 * 4;
constexpr uint32_t kSfaSmemBytes = kSfaOffBar + 512;
static_assert(kSfaOffK % 1024 == 0 && kSfaOffV % 1024 == 0 && kSfaOffP % 1024 == 0, "operand alignment");
static_assert(kSfaSmemBytes <= 232448, "shared memory");

// setmaxnreg.inc only ever gets registers that warps of the SAME CTA have released and blocks (for
// good) until it has them: what the softmax warps ask for must fit into what the others give back.
constexpr int kSfaLaunchRegs = 80;   // 65536 / 768 threads, rounded down to a multiple of 8
constexpr int kSfaRegsLow = 56, kSfaRegsHigh = 168;
static_assert((kSfaRegsHigh - kSfaLaunchRegs) * (kSfaThreads / 32 - kSfaSoftWarp0) <=
                  (kSfaLaunchRegs - kSfaRegsLow) * kSfaCopyWarp0,
              "setmaxnreg: more registers requested than released");
static_assert(kSfaLaunchRegs * kSfaThreads <= 65536, "register file");

constexpr uint32_t kTmO = 0, kTmS = 256;
constexpr float kSfaRescaleTau = 8.f;  // log2 units: the running reference only moves when exceeded by this

struct SfaSm100Args {
  SfaDev p;
  int32_t* status;
  uint32_t idesc_qk, idesc_pv;
  float scale_log2;  // scale * log2(e)
  int32_t is_bf16;
  const int2* nvalid;       // [items] .x participating slots, .y first entry in key_list (pre-pass output)
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

// Development aid, compiled only with -DDSA_SFA_PROFILE: cycle sums per role of the first cluster
// (slot = role * 8 + counter, odd CTA + 64), read back with dsa_debug_sfa_profile().
#ifdef DSA_SFA_PROFILE
__device__ long long g_sfa_prof[128];
#define SFA_PROF_DECL long long pacc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long pt = clock64()
#define SFA_PROF(i) do { const long long pn = clock64(); pacc[i] += pn - pt; pt = pn; } while (0)
#define SFA_PROF_STORE(role, cond) do { if (blockIdx.x < 2 && (cond)) { \
    for (int pi = 0; pi < 8; ++pi) g_sfa_prof[(blockIdx.x & 1) * 64 + (role) * 8 + pi] = pacc[pi]; } } while (0)
#else
#define SFA_PROF_DECL
#define SFA_PROF(i)
#define SFA_PROF_STORE(role, cond)
#endif

// Pre-pass: one warp per query row.  Writes the physical KV rows of the slots that take part, in
// slot order, and their count.  A slot whose paged block is absent inside the valid length takes
// part as a zero row, like the reference's un-paged cache
// (sparse_flash_attention_triton.py:1012-1033): it gets the row number `oob_row` (= the number of
// KV rows), which the gather loads as zeros.
__global__ void __launch_bounds__(128) sfa_compact_kernel(SfaDev p, int2* __restrict__ nvalid,
                                                          int32_t* __restrict__ key_list, int32_t split,
                                                          int32_t part_keys, int32_t oob_row) {
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
        if (tok >= 0) {
          prow = key_row(p.seq, ri, tok);
          if (prow < 0 || prow >= oob_row) prow = oob_row;
        }
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
                     const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_qr,
                     const SfaSm100Args a) {
  extern __shared__ __align__(1024) unsigned char sfa_sm[];
  unsigned char* q_s = sfa_sm + kSfaOffQ;
  unsigned char* k_s = sfa_sm + kSfaOffK;
  unsigned char* v_s = sfa_sm + kSfaOffV;
  unsigned char* p_s = sfa_sm + kSfaOffP;
  float* xm = reinterpret_cast<float*>(sfa_sm + kSfaOffX);   // [2][128] running-maximum exchange
  float* xs = xm + 256;                                       // [128] row-sum exchange
  uint64_t* bars = reinterpret_cast<uint64_t*>(sfa_sm + kSfaOffBar);
  // K barriers are indexed [slot * 3 + issuer]: every issuer's three feature blocks are handed over
  // and released on their own.
  uint64_t* k_full = bars;         // [6] gather -> QK issuer / relay                 (tx bytes)
  uint64_t* k_empty = bars + 6;    // [6] blocks read by the issuer's MMAs (commit) and by the four copier warps -> K producers
  uint64_t* k_ready = bars + 12;   // [6] even CTA only: the odd CTA's blocks have landed
  uint64_t* v_full = bars + 18;    // [2] own copier warps (4 arrivals + 1 arming) and the peer's st.async bytes -> PV issuer / relay
  uint64_t* v_empty = bars + 20;   // [2] PV of the tile done -> V copier              (commit, both CTAs)
  uint64_t* v_ready = bars + 22;   // [2] even CTA only: the odd CTA's V slot has landed
  uint64_t* s_full = bars + 24;    // [2] all three partial products done -> softmax   (commit x 3, both CTAs)
  uint64_t* s_empty = bars + 26;   // [2] even CTA only: softmax warps of both CTAs hold S in registers
  uint64_t* p_full = bars + 28;    // [2] even CTA only: P stored (O rescaled) in both CTAs
  uint64_t* p_empty = bars + 30;   // [2] PV done -> softmax                           (commit, both CTAs)
  uint64_t* q_full = bars + 32;    // this CTA's Q has landed (tx bytes)
  uint64_t* q_ready = bars + 33;   // even CTA only: the odd CTA's Q has landed
  uint64_t* q_empty = bars + 34;   // all QK issuers are through with the token        (commit x 3, both CTAs)
  uint64_t* o_free = bars + 35;    // even CTA only: epilogue warps of both CTAs have read O
  uint64_t* x_bar = bars + 36;     // softmax warps: exchange buffer written
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 37);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 38);
  static_assert(39 * 8 <= 512, "barrier area");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int32_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  const bool misaligned = (ptx::smem_u32(sfa_sm) & 1023u) != 0;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 6; ++i) {
      ptx::mbar_init(&k_full[i], 1); ptx::mbar_init(&k_empty[i], 5); ptx::mbar_init(&k_ready[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&v_full[i], 5); ptx::mbar_init(&v_empty[i], 1); ptx::mbar_init(&v_ready[i], 1);
      ptx::mbar_init(&s_full[i], kSfaQkLanes); ptx::mbar_init(&s_empty[i], 8);
      ptx::mbar_init(&p_full[i], 8); ptx::mbar_init(&p_empty[i], 1);
    }
    ptx::mbar_init(q_full, 1);
    ptx::mbar_init(q_ready, 1);
    ptx::mbar_init(q_empty, kSfaQkLanes);
#ifdef DSA_EXP_PRODONLY
    ptx::mbar_init(o_free, kSfaKWarps);
    reinterpret_cast<volatile int*>(xs)[0] = 0; reinterpret_cast<volatile int*>(xs)[1] = 0;
#else
    ptx::mbar_init(o_free, 8);
#endif
    ptx::mbar_init(x_bar, 4);
    *abort_flag = misaligned ? 1 : 0;
    ptx::mbar_fence_init();
  }
  if (warp == kSfaQkWarp0) {
    ptx::tmem_alloc_pair(tmem_slot, 512);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // the peer's barriers must exist before anything is sent to it
  ptx::cluster_arrive();
  ptx::cluster_wait();
  const uint32_t tmem = *tmem_slot;

  const int32_t n1 = a.p.n1;                   // real heads (<= 128); rows past them carry zero queries
  auto item_tiles = [&](int32_t item) -> int32_t { return (a.nvalid[item].x + kSfaBK - 1) / kSfaBK; };

  if (warp < kSfaSoftWarp0) {
    // registers: kSfaLaunchRegs per thread at launch; producers and issuers give some back, the
    // softmax warps take them (whole warpgroups of four warps change together)
    if (warp < kSfaCopyWarp0) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kSfaRegsLow));
    if (*abort_flag) {
      // nothing started: fall through to the teardown
    } else if (warp < kSfaKWarps) {
      // ------------------------------------------------------------------ K gather producers
      // Three warps per QK^T issuer: 8 row groups (4 of this CTA's 32 keys each) x the issuer's 3
      // column blocks = 24 gather4 loads of 512 bytes per tile, dealt out over the three warps.
      // Measured in this kernel: the lanes of a warp issue one after the other, ~220 cycles per
      // load; warps issue in parallel until the SM's TMA unit saturates at one load per ~18 cycles
      // (28 B/clk, bulk copies included) - which is why nothing but these loads goes through it.
      const int qi = warp / 3;                           // the issuer this warp feeds
      const int gw = warp - qi * 3;
      const int o = gw + 3 * lane;
      const bool active = o < 24;
      const int grp = o / 3, blk = 3 * qi + (o - grp * 3);
      const int key0 = (int)rank * kSfaHalfBK + grp * 4;   // first key (within the tile) of this load
      const int32_t x = blk < 8 ? blk * 64 : 0;
      unsigned char* slot0 = k_s + blk * kSfaKBlk + grp * 512;
      uint64_t* full = k_full + qi;                      // slot s: full[s * 3]
      uint64_t* empty = k_empty + qi;
      if (lane == 0) { ptx::prefetch_tmap(&tmap_kn); ptx::prefetch_tmap(&tmap_kr); }
      // The row numbers of a tile come from global memory (the pre-pass list); they are fetched one
      // tile ahead so that their latency never sits between a freed slot and the gather.
      struct TilePos { int32_t item, t, ntiles, nvalid, off; };
      auto first_from = [&](int32_t item) -> TilePos {
        for (; item < a.items; item += n_clusters) {
          const int2 d = a.nvalid[item];
          if (d.x > 0) return TilePos{item, 0, (d.x + kSfaBK - 1) / kSfaBK, d.x, d.y};
        }
        return TilePos{a.items, 0, 0, 0, 0};
      };
      auto load_rows = [&](const TilePos& tp, int32_t* r) {
        const int32_t* list = a.key_list + tp.off;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int32_t k = tp.t * kSfaBK + key0 + i;
          // keys past the end of the row re-read the tile's first key (masked by the softmax)
          r[i] = (active && tp.item < a.items) ? list[k < tp.nvalid ? k : tp.t * kSfaBK] : 0;
        }
      };
      uint32_t n_tile = 0;
      bool ok = true;
      SFA_PROF_DECL;
      TilePos cur = first_from(cluster_id);
      int32_t rc[4], rn[4];
      load_rows(cur, rc);
      while (cur.item < a.items && ok) {
        TilePos nxt = cur;
        if (++nxt.t >= nxt.ntiles) nxt = first_from(cur.item + n_clusters);
        load_rows(nxt, rn);
        const uint32_t s = n_tile & 1, use = n_tile >> 1;
        SFA_PROF(0);
#ifndef DSA_EXP_PRODONLY
        ok = ptx::mbar_wait_warp(&empty[s * 3], (use & 1) ^ 1, abort_flag);
#else
        // timing experiment: no consumer; a slot is re-armed once its previous load has landed
        if (lane == 0 && use > 0) ok = ptx::mbar_wait(&full[s * 3], (use - 1) & 1, abort_flag);
#endif
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        SFA_PROF(1);
        if (gw == 0 && lane == 0) ptx::mbar_arrive_expect_tx(&full[s * 3], kSfaKSub);
        __syncwarp();
        SFA_PROF(3);
        // the tensor map is named directly in each call (a map chosen through a per-lane pointer
        // costs an address conversion per load)
        if (active) {
#ifdef DSA_EXP_ONEMAP
          if (blk == 8) ptx::tma_gather4_2d(slot0 + s * kSfaKSlot, &tmap_kn, &full[s * 3], 0, rc[0], rc[1], rc[2], rc[3]);
#else
          if (blk == 8) ptx::tma_gather4_2d(slot0 + s * kSfaKSlot, &tmap_kr, &full[s * 3], 0, rc[0], rc[1], rc[2], rc[3]);
#endif
          else ptx::tma_gather4_2d(slot0 + s * kSfaKSlot, &tmap_kn, &full[s * 3], x, rc[0], rc[1], rc[2], rc[3]);
        }
        SFA_PROF(4);
        __syncwarp();
        SFA_PROF(2);
        ++n_tile;
        cur = nxt;
#pragma unroll
        for (int i = 0; i < 4; ++i) rc[i] = rn[i];
      }
#ifdef DSA_EXP_PRODONLY
      // drain: the last loads of both slots must have landed before the CTA may exit
      if (lane == 0) {
        for (uint32_t back = 1; back <= 2 && back <= n_tile; ++back) {
          const uint32_t n = n_tile - back;
          ptx::mbar_wait(&full[(n & 1) * 3], (n >> 1) & 1, abort_flag);
        }
      }
      __syncwarp();
      if (lane == 0) { ptx::mbar_arrive(o_free); atomicAdd(reinterpret_cast<int*>(xs) + 1, 1); if (reinterpret_cast<volatile int*>(xs)[1] == kSfaKWarps) *reinterpret_cast<volatile int*>(xs) = 1; }
#endif
      SFA_PROF_STORE(0, lane == 0 && warp == 0);
#ifdef DSA_EXP_PRODONLY
    } else if (true) {
#if DSA_EXP_PRODONLY == 2
      ptx::mbar_wait_warp(o_free, 0, abort_flag);          // o_free: 8 arrivals... re-initialised below to 9
#elif DSA_EXP_PRODONLY == 3
      while (*reinterpret_cast<volatile int*>(xs) == 0) __nanosleep(500);
#elif DSA_EXP_PRODONLY >= 4
      // waits that give up as soon as the producers of this CTA are done (timing experiments only)
      auto fwait = [&](uint64_t* bar, uint32_t par) -> bool {
        bool got = true;
        while (!ptx::mbar_try_wait(bar, par)) { if (*reinterpret_cast<volatile int*>(xs) != 0) { got = false; break; } }
        return __all_sync(0xffffffffu, got);
      };
#endif
#if DSA_EXP_PRODONLY == 4
      // one warp per CTA keeps issuing tcgen05.commit (even CTA, multicast) and both wait for it
      if (warp == 12) {
        uint32_t ph = 0;
        while (*reinterpret_cast<volatile int*>(xs) == 0) {
          if (rank == 0 && ptx::elect_one()) ptx::mma_commit_pair(&s_full[0]);   // count 3 -> needs 3 commits per phase
          if (rank == 0 && ptx::elect_one()) ptx::mma_commit_pair(&s_full[0]);
          if (rank == 0 && ptx::elect_one()) ptx::mma_commit_pair(&s_full[0]);
          __syncwarp();
          if (!fwait(&s_full[0], ph & 1)) break;
          ++ph;
          __nanosleep(200);
        }
      } else { while (*reinterpret_cast<volatile int*>(xs) == 0) __nanosleep(500); }
#elif DSA_EXP_PRODONLY == 5
      // four warps ping-pong through shared memory + an mbarrier (like the softmax exchange)
      if (warp >= 16 && warp < 20) {
        uint32_t ph = 0;
        const int L = (warp - 16) * 32 + lane;
        while (*reinterpret_cast<volatile int*>(xs) == 0) {
          xm[L] = (float)ph;
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(x_bar);
          if (!fwait(x_bar, ph & 1)) break;
          ++ph;
          if (xm[L ^ 64] < 0.f) break;
          __nanosleep(200);
        }
      } else { while (*reinterpret_cast<volatile int*>(xs) == 0) __nanosleep(500); }
#elif DSA_EXP_PRODONLY == 6
      // the odd CTA's warp 12 keeps sending relaxed remote arrivals to the even CTA's warp 12, which waits for them
      if (warp == 12) {
        uint32_t ph = 0;
        const uint32_t rb = ptx::map_to_rank(q_ready, 0);
        while (*reinterpret_cast<volatile int*>(xs) == 0) {
          if (rank != 0) { if (ptx::elect_one()) ptx::mbar_arrive_remote_relaxed(rb, 0u); __syncwarp(); __nanosleep(400); }
          else { if (!fwait(q_ready, ph & 1)) break; ++ph; }
        }
      } else { while (*reinterpret_cast<volatile int*>(xs) == 0) __nanosleep(500); }
#elif DSA_EXP_PRODONLY == 8 || DSA_EXP_PRODONLY == 9
      // idle warps watch the very barriers the gathers complete on (8: five warps, all lanes; 9: one lane of one warp)
      if ((DSA_EXP_PRODONLY == 8 && (warp == 12 || (warp >= 16 && warp < 20))) || (DSA_EXP_PRODONLY == 9 && warp == 12)) {
        for (uint32_t n = 0; *reinterpret_cast<volatile int*>(xs) == 0; ++n) {
          const uint32_t b = n & 1, use = n >> 1;
          bool got = true;
          if (DSA_EXP_PRODONLY == 8 || lane == 0) {
            for (int i = 0; i < 3 && got; ++i)
              while (!ptx::mbar_try_wait(&k_full[b * 3 + i], use & 1)) { if (*reinterpret_cast<volatile int*>(xs) != 0) { got = false; break; } }
          }
          if (!__all_sync(0xffffffffu, got)) break;
        }
      } else { while (*reinterpret_cast<volatile int*>(xs) == 0) __nanosleep(500); }
#elif DSA_EXP_PRODONLY == 7
      // four warps keep storing to global memory (epilogue-like, 32-byte stores to rows 1 KB apart)
      if (warp >= 16 && warp < 20) {
        const int L = (warp - 16) * 32 + lane;
        unsigned char* o = (unsigned char*)a.p.out + ((int64_t)(cluster_id * 2 + rank) * 128 + L) * 1024;
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int it = 0;
        while (*reinterpret_cast<volatile int*>(xs) == 0) { ptx::st_global_v8(o + (it & 31) * 32, w); ++it; if ((it & 31) == 0) __nanosleep(300); }
      } else { while (*reinterpret_cast<volatile int*>(xs) == 0) __nanosleep(500); }
#endif
#endif
    } else if (warp == kSfaQWarp) {
      // ------------------------------------------------------------------ Q loader
      // Per token: this CTA's 64 heads x 576 features into shared memory (nine 64 x 64 boxes; heads
      // past n1 read as zeros), as soon as all QK^T issuers are through with the previous token.
      // The other lanes pull the next token's rows into L2 meanwhile.
      uint32_t n_tok = 0;
      bool ok = true;
      const uint32_t q_ready_lead = ptx::map_to_rank(q_ready, 0);
      if (lane == 0) { ptx::prefetch_tmap(&tmap_q); ptx::prefetch_tmap(&tmap_qr); }
      const int32_t h0 = (int32_t)rank * kSfaCtaHeads;
      const int32_t hn = min(kSfaCtaHeads, n1 - h0);     // this CTA's real heads (may be <= 0)
      for (int32_t item = cluster_id; item < a.items && ok; item += n_clusters) {
        if (item_tiles(item) == 0) continue;
        const int32_t row = kSplit ? item / a.split : item;
        if (lane == 0) {
          ok = ptx::mbar_wait(q_empty, (n_tok & 1) ^ 1, abort_flag);
          if (ok) {
            ptx::mbar_arrive_expect_tx(q_full, kSfaQBytes);
#pragma unroll 1
            for (int f = 0; f < 9; ++f)
              ptx::tma_load_3d(q_s + f * kSfaQBlk, f < 8 ? &tmap_q : &tmap_qr, q_full, f < 8 ? f * 64 : 0, h0, row);
            if (rank != 0) {
              ok = ptx::mbar_wait(q_full, n_tok & 1, abort_flag);
              if (ok) ptx::mbar_arrive_remote_relaxed(q_ready_lead, 0u);
            }
          }
        } else if (hn > 0) {
          int32_t nitem = item + n_clusters;
          while (nitem < a.items && a.nvalid[nitem].x == 0) nitem += n_clusters;
          if (nitem < a.items) {
            const int32_t nrow = kSplit ? nitem / a.split : nitem;
            const unsigned char* qn = (const unsigned char*)a.p.query + ((int64_t)nrow * n1 + h0) * (kSfaDv * 2);
            const unsigned char* qr = (const unsigned char*)a.p.query_rope + ((int64_t)nrow * n1 + h0) * 128;
            for (int32_t i = lane - 1; i < hn * 8; i += 31) ptx::prefetch_l2(qn + (int64_t)i * 128);
            for (int32_t i = lane - 1; i < hn; i += 31) ptx::prefetch_l2(qr + (int64_t)i * 128);
          }
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        ++n_tok;
      }
    } else if (warp >= kSfaQkWarp0 && warp < kSfaPvWarp) {
      // ------------------------------------------------------------------ QK^T issuers (even CTA) / K relays (odd CTA)
      // Issuer i multiplies feature blocks 3i..3i+2 of every tile into its own partial S; the
      // softmax adds the three partials.  One thread issues a short (N = 64) MMA only every 60-90
      // cycles, three keep the tensor pipe busy.  The loop is warp-uniform (every lane waits) and
      // only the MMA and the commits are issued by one elected lane.
      const uint32_t qi = warp - kSfaQkWarp0;
      uint32_t n_tile = 0, n_tok = 0;
      bool ok = true;
      const uint32_t q_addr = ptx::smem_u32(q_s) + qi * 3 * kSfaQBlk;
      const uint32_t k_addr = ptx::smem_u32(k_s) + qi * kSfaKSub;
      const uint32_t k_ready_lead = ptx::map_to_rank(k_ready, 0);
      SFA_PROF_DECL;
      for (int32_t item = cluster_id; item < a.items && ok; item += n_clusters) {
        const int32_t ntiles = item_tiles(item);
        if (ntiles == 0) continue;
        SFA_PROF(0);
        if (rank == 0) {
          ok = ptx::mbar_wait_warp(q_full, n_tok & 1, abort_flag) && ptx::mbar_wait_cluster_warp(q_ready, n_tok & 1, abort_flag);
        }
        SFA_PROF(5);
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          const uint32_t b = n_tile & 1, use = n_tile >> 1, kb = b * kSfaQkLanes + qi;
          SFA_PROF(0);
          ok = ptx::mbar_wait_warp(&k_full[kb], use & 1, abort_flag);
          if (!ok) break;
          SFA_PROF(1);
          if (rank != 0) {
            // relaxed: the blocks were written by the TMA unit and are complete once the barrier
            // says so; nothing of this thread's own has to be published
            if (ptx::elect_one()) ptx::mbar_arrive_remote_relaxed(k_ready_lead + kb * 8, 0u);
            __syncwarp();
            continue;
          }
          ok = ptx::mbar_wait_cluster_warp(&k_ready[kb], use & 1, abort_flag);
          SFA_PROF(2);
          ok = ok && ptx::mbar_wait_cluster_warp(&s_empty[b], (use & 1) ^ 1, abort_flag);
          if (!ok) break;
          SFA_PROF(3);
          ptx::tc_fence_after();
          if (ptx::elect_one()) {
#pragma unroll
            for (int f = 0; f < 3; ++f) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                const uint64_t ad = ptx::desc_kmajor_sw128(q_addr + f * kSfaQBlk + kk * 32);
                const uint64_t bd = ptx::desc_kmajor_sw128(k_addr + b * kSfaKSlot + f * kSfaKBlk + kk * 32);
                ptx::mma_ss_pair(tmem + kTmS + kb * 32, ad, bd, a.idesc_qk, (f | kk) ? 1u : 0u);
              }
            }
            ptx::mma_commit_pair(&s_full[b]);
            ptx::mma_commit_pair(&k_empty[kb]);
          }
          __syncwarp();
          SFA_PROF(4);
        }
        // the token's Q may be replaced once every issuer's products have completed
        if (ok && rank == 0 && ptx::elect_one()) ptx::mma_commit_pair(q_empty);
        __syncwarp();
        ++n_tok;
      }
      SFA_PROF_STORE(2, lane == 0 && qi == 0);
    } else if (warp >= kSfaCopyWarp0) {
      // ------------------------------------------------------------------ V copiers
      // The value operand of a tile (all 64 keys x this CTA's 256 value columns) is not gathered
      // again - the TMA unit is the busiest part of this kernel.  Every CTA already holds its own
      // 32 keys with all columns in its K slot: these 128 threads copy the four column blocks that
      // this CTA owns into its own V slot (plain loads and stores) and the four that the peer owns
      // into the peer's V slot (st.async: the bytes are counted on the peer's barrier when they
      // land, the sender does not wait), rows 32*rank.. of every block; 16 chunks of 16 bytes per
      // thread.  Byte offsets inside 4 KB are kept, so the 128-byte swizzle pattern carries over.
      const int tid = (warp - kSfaCopyWarp0) * 32 + lane;
      const uint32_t peer = rank ^ 1u;
      const uint32_t v_peer = ptx::map_to_rank(v_s, peer);
      const uint32_t v_full_peer = ptx::map_to_rank(v_full, peer);
      uint32_t n_tile = 0;
      bool ok = true;
      SFA_PROF_DECL;
      for (int32_t item = cluster_id; item < a.items && ok; item += n_clusters) {
        const int32_t ntiles = item_tiles(item);
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          const uint32_t b = n_tile & 1, use = n_tile >> 1;
          SFA_PROF(0);
          // V slot b is free in both CTAs once the product that read it has completed
          ok = ptx::mbar_wait_warp(&v_empty[b], (use & 1) ^ 1, abort_flag);
          if (!ok) break;
          SFA_PROF(1);
          // the peer's half of my V slot: 16 KB of transaction bytes
#ifdef DSA_EXP_NOCOPY
          if (tid == 0) ptx::mbar_arrive(&v_full[b]);
#else
          if (tid == 0) ptx::mbar_arrive_expect_tx(&v_full[b], kSfaVSlot / 2);
#endif
          ok = ptx::mbar_wait_warp(&k_full[b * 3], use & 1, abort_flag) &&
               ptx::mbar_wait_warp(&k_full[b * 3 + 1], use & 1, abort_flag) &&
               ptx::mbar_wait_warp(&k_full[b * 3 + 2], use & 1, abort_flag);
          if (!ok) break;
          SFA_PROF(2);
          const unsigned char* ksrc = k_s + b * kSfaKSlot;
          const uint32_t vdst = b * kSfaVSlot + rank * kSfaKBlk;     // rows 32*rank.. of a V block
#ifndef DSA_EXP_NOCOPY
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            // half 0: the four blocks this CTA owns (local), half 1: the four the peer owns (remote)
            const int owner = half == 0 ? (int)rank : (int)peer;
            uint4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int q = i * 128 + tid;                      // 0..1023: chunk within the four blocks
              const int pblk = q >> 8, within = q & 255;
              const int fblk = 4 * (pblk >> 1) + 2 * owner + (pblk & 1);
              v[i] = *reinterpret_cast<const uint4*>(ksrc + fblk * kSfaKBlk + within * 16);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int q = i * 128 + tid;
              const int pblk = q >> 8, within = q & 255;
              const uint32_t off = vdst + pblk * kSfaVBlk + within * 16;
              if (half == 0) *reinterpret_cast<uint4*>(v_s + off) = v[i];
              else ptx::st_async_v4(v_peer + off, v[i], v_full_peer + b * 8);
            }
          }
#endif
          SFA_PROF(3);
          // the K slot has been read (the loads have returned): its producers may refill it; the
          // local rows are made visible to the tensor core's reads before the arrival says so
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane < 3) ptx::mbar_arrive(&k_empty[b * 3 + lane]);
          if (lane == 0) ptx::mbar_arrive(&v_full[b]);
          SFA_PROF(4);
        }
      }
      SFA_PROF_STORE(1, tid == 0);
    } else if (warp == kSfaPvWarp) {
      // ------------------------------------------------------------------ PV issuer (even CTA) / V relay (odd CTA)
      uint32_t n_tile = 0, n_tok = 0;
      bool ok = true;
      const uint32_t p_addr = ptx::smem_u32(p_s), v_addr = ptx::smem_u32(v_s);
      const uint32_t v_ready_lead = ptx::map_to_rank(v_ready, 0);
      SFA_PROF_DECL;
      for (int32_t item = cluster_id; item < a.items && ok; item += n_clusters) {
        const int32_t ntiles = item_tiles(item);
        if (ntiles == 0) continue;
        // the previous token's O has been read out in both CTAs
        SFA_PROF(0);
        if (rank == 0) ok = ptx::mbar_wait_cluster_warp(o_free, (n_tok & 1) ^ 1, abort_flag);
        SFA_PROF(5);
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          const uint32_t b = n_tile & 1, use = n_tile >> 1;
          SFA_PROF(0);
          ok = ptx::mbar_wait_cluster_warp(&v_full[b], use & 1, abort_flag);
          if (!ok) break;
          SFA_PROF(1);
          if (rank != 0) {
            // the peer's rows arrived through the generic proxy: order them before the tensor core's
            // reads of this CTA's shared memory, then tell the issuer
            if (ptx::elect_one()) {
              ptx::fence_proxy_async_smem();
              ptx::mbar_arrive_remote_relaxed(v_ready_lead + b * 8, 0u);
            }
            __syncwarp();
            continue;
          }
          ok = ptx::mbar_wait_cluster_warp(&v_ready[b], use & 1, abort_flag);
          SFA_PROF(2);
          ok = ok && ptx::mbar_wait_cluster_warp(&p_full[b], use & 1, abort_flag);
          if (!ok) break;
          SFA_PROF(3);
          ptx::tc_fence_after();
          if (ptx::elect_one()) {
            ptx::fence_proxy_async_smem();   // the V rows the peer stored into this CTA (generic proxy)
#pragma unroll
            for (int ks = 0; ks < kSfaBK / 16; ++ks) {
              const uint64_t ad = ptx::desc_kmajor_sw128(p_addr + b * kSfaPBuf + ks * 32);
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const uint64_t bd = ptx::desc_mnmajor_sw128(v_addr + b * kSfaVSlot + j * 2 * kSfaVBlk + ks * 16 * 128,
                                                            kSfaVBlk, 1024);
                ptx::mma_ss_pair(tmem + kTmO + j * 128, ad, bd, a.idesc_pv, (t == 0 && ks == 0) ? 0u : 1u);
              }
            }
            ptx::mma_commit_pair(&p_empty[b]);
            ptx::mma_commit_pair(&v_empty[b]);
          }
          __syncwarp();
          SFA_PROF(4);
        }
        ++n_tok;
      }
      SFA_PROF_STORE(3, lane == 0);
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSfaRegsHigh));
#ifdef DSA_EXP_PRODONLY
#if DSA_EXP_PRODONLY == 2
    ptx::mbar_wait_warp(o_free, 0, abort_flag);
#elif DSA_EXP_PRODONLY >= 3
    while (*reinterpret_cast<volatile int*>(xs) == 0) __nanosleep(500);
#endif
    if (false) {
#else
    if (!*abort_flag) {
#endif
      // ------------------------------------------------------------------ softmax + epilogue
      const int quarter = warp & 3;
      const int L = quarter * 32 + lane;            // TMEM lane
      const int hl = L & 63, half = L >> 6;         // head within this CTA; which half of N this lane holds
      const int32_t hg = (int32_t)rank * kSfaCtaHeads + hl;
      const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
      const uint32_t s_empty_lead = ptx::map_to_rank(s_empty, 0);
      const uint32_t p_full_lead = ptx::map_to_rank(p_full, 0);
      const uint32_t o_free_lead = ptx::map_to_rank(o_free, 0);
      uint32_t n_tile = 0, n_x = 0;
      bool ok = true;
      SFA_PROF_DECL;
      // waits are warp-wide: the tcgen05 loads / stores that follow are warp-collective and must
      // never run with part of a warp gone
      auto wait_w = [&](uint64_t* bar, uint32_t parity) -> bool { return ptx::mbar_wait_warp(bar, parity, abort_flag); };
      // One arrival per warp on a barrier of the even CTA.  From the odd CTA it is a relaxed remote
      // arrival: a cluster-scope release costs ~1000 cycles here, and what the arrival announces has
      // already been made visible by the fences before it (tcgen05.wait + tcgen05 fence for tensor
      // memory, fence.proxy.async for the P rows, which lie in this CTA's own shared memory).
      auto signal_lead = [&](uint64_t* local, uint32_t remote) {
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) ptx::mbar_arrive(local);
          else ptx::mbar_arrive_remote_relaxed(remote, 0u);
        }
      };
      // value of the head's other thread (lane L ^ 64, another warp) through shared memory
      auto exchange = [&](float* buf, float v, float& other) -> bool {
        buf[L] = v;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(x_bar);
        const bool got = wait_w(x_bar, n_x & 1);
        ++n_x;
        other = buf[L ^ 64];
        return got;
      };
      for (int32_t item = cluster_id; item < a.items && ok; item += n_clusters) {
        const int32_t nvalid = a.nvalid[item].x;
        const int32_t ntiles = (nvalid + kSfaBK - 1) / kSfaBK;
        const int32_t row = kSplit ? item / a.split : item;
        // this lane's output columns: j * 256 + half * 128 + 0..127 for j = 0, 1
        unsigned char* out_row = (unsigned char*)a.p.out + (((int64_t)row * n1 + hg) * kSfaDv + half * 128) * 2;
        float* part_row = kSplit ? a.part_o + ((int64_t)item * kSfaHeads + hg) * kSfaDv + half * 128 : nullptr;
        if (ntiles == 0) {
          if constexpr (kSplit) {
            // an empty part: the merge skips it
            if (half == 0) { a.part_m[(int64_t)item * kSfaHeads + hg] = 0.f; a.part_l[(int64_t)item * kSfaHeads + hg] = 0.f; }
          } else if (hg < n1) {
            // nothing visible: zeros in all three outputs
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
              for (int c = 0; c < 16; ++c) reinterpret_cast<uint4*>(out_row + j * 512)[c] = make_uint4(0, 0, 0, 0);
            if (half == 0 && a.p.return_lse) {
              a.p.softmax_max[(int64_t)row * n1 + hg] = 0.f;
              a.p.softmax_sum[(int64_t)row * n1 + hg] = 0.f;
            }
          }
          continue;
        }
        float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f, l_tot = 0.f;
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          const uint32_t b = n_tile & 1, use = n_tile >> 1;
          const int32_t cnt = min(kSfaBK, nvalid - t * kSfaBK) - half * kSfaHalfBK;   // valid keys among this lane's 32
          SFA_PROF(7);
          ok = wait_w(&s_full[b], use & 1);
          if (!ok) break;
          SFA_PROF(0);
          ptx::tc_fence_after();
          float sc[kSfaHalfBK];
#ifdef DSA_EXP_NOSOFT
          for (int k = 0; k < kSfaHalfBK; ++k) sc[k] = 0.f;
          if (false)
#endif
          {
            // the three issuers' partial products
            float s1[kSfaHalfBK], s2[kSfaHalfBK];
            ptx::tmem_ld_x32(lane_addr + kTmS + (b * kSfaQkLanes) * 32, reinterpret_cast<uint32_t*>(sc));
            ptx::tmem_ld_x32(lane_addr + kTmS + (b * kSfaQkLanes + 1) * 32, reinterpret_cast<uint32_t*>(s1));
            ptx::tmem_ld_x32(lane_addr + kTmS + (b * kSfaQkLanes + 2) * 32, reinterpret_cast<uint32_t*>(s2));
            ptx::tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < kSfaHalfBK; ++k) sc[k] = (sc[k] + s1[k]) + s2[k];
          }
          ptx::tc_fence_before();
          signal_lead(&s_empty[b], s_empty_lead + b * 8);
          SFA_PROF(1);
          // ---- softmax in the log2 domain; keys past `cnt` are padding
          if (cnt >= kSfaHalfBK) {
#pragma unroll
            for (int k = 0; k < kSfaHalfBK; ++k) sc[k] *= a.scale_log2;
          } else {
#pragma unroll
            for (int k = 0; k < kSfaHalfBK; ++k) sc[k] = k < cnt ? sc[k] * a.scale_log2 : -INFINITY;
          }
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int k = 0; k < kSfaHalfBK; k += 4) {
            mx4[0] = fmaxf(mx4[0], sc[k]); mx4[1] = fmaxf(mx4[1], sc[k + 1]);
            mx4[2] = fmaxf(mx4[2], sc[k + 2]); mx4[3] = fmaxf(mx4[3], sc[k + 3]);
          }
          float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])), mx_other;
          SFA_PROF(2);
          ok = exchange(xm + b * 128, mx, mx_other);
          if (!ok) break;
          SFA_PROF(3);
          mx = fmaxf(mx, mx_other);       // the tile's maximum for this head (the first half always has a valid key)
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
          for (int k = 0; k < kSfaHalfBK; k += 4) {
            sc[k] = ex2(sc[k] - m_ref); sc[k + 1] = ex2(sc[k + 1] - m_ref);
            sc[k + 2] = ex2(sc[k + 2] - m_ref); sc[k + 3] = ex2(sc[k + 3] - m_ref);
            sum4[0] += sc[k]; sum4[1] += sc[k + 1]; sum4[2] += sc[k + 2]; sum4[3] += sc[k + 3];
          }
          l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
          if (ntiles == 1) {
            // a single tile holds the whole row: normalise before rounding, as the golden does
            float l_other;
            ok = exchange(xs, l, l_other);
            if (!ok) break;
            l_tot = l + l_other;
            const float inv = 1.f / l_tot;
#pragma unroll
            for (int k = 0; k < kSfaHalfBK; ++k) sc[k] *= inv;
          }
          // ---- P (and, rarely, a rescaled O) once the product that last read this P buffer has finished
          SFA_PROF(2);
          ok = wait_w(&p_empty[b], (use & 1) ^ 1);
          if (!ok) break;
          SFA_PROF(4);
          if (__any_sync(0xffffffffu, rescale)) {
            // O must be quiescent: the previous tile's product (other P buffer) has to be complete too
            const uint32_t prev = n_tile - 1;
            ok = wait_w(&p_empty[prev & 1], (prev >> 1) & 1);
            if (!ok) break;
            ptx::tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 8; ++c) {
              uint32_t o[32];
              ptx::tmem_ld_x32(lane_addr + kTmO + c * 32, o);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              ptx::tmem_st_x32(lane_addr + kTmO + c * 32, o);
            }
            ptx::tmem_st_wait();
          }
#ifdef DSA_EXP_NOSOFT
          if (false)
#endif
          {
            // row hl of the K-major, 128-byte-swizzled A operand: keys half*32 .. +31 are the 16-byte
            // chunks half*4 .. +3 of the row
            unsigned char* prow = p_s + b * kSfaPBuf + hl * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 w;
              w.x = pack2(sc[8 * c], sc[8 * c + 1], a.is_bf16);
              w.y = pack2(sc[8 * c + 2], sc[8 * c + 3], a.is_bf16);
              w.z = pack2(sc[8 * c + 4], sc[8 * c + 5], a.is_bf16);
              w.w = pack2(sc[8 * c + 6], sc[8 * c + 7], a.is_bf16);
              *reinterpret_cast<uint4*>(prow + (((half * 4 + c) ^ (hl & 7)) << 4)) = w;
            }
          }
          ptx::fence_proxy_async_smem();
          ptx::tc_fence_before();
          signal_lead(&p_full[b], p_full_lead + b * 8);
          SFA_PROF(5);
        }
        if (!ok) break;
        SFA_PROF(7);
        // ---- epilogue: wait for the last product, normalise, store
        {
          const uint32_t last = n_tile - 1;
          ok = wait_w(&p_empty[last & 1], (last >> 1) & 1);
          if (!ok) break;
        }
        ptx::tc_fence_after();
        if (ntiles > 1) {
          float l_other;
          ok = exchange(xs, l, l_other);
          if (!ok) break;
          l_tot = l + l_other;
        }
        const float inv = ntiles == 1 ? 1.f : 1.f / l_tot;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          // c = j * 4 + chunk: accumulator columns c*32 .. +31 = value columns j*256 + half*128 + chunk*32 ..
          uint32_t o[32];
          ptx::tmem_ld_x32(lane_addr + kTmO + c * 32, o);
          ptx::tmem_ld_wait();
          const int col = (c >> 2) * 256 + (c & 3) * 32;   // relative to half * 128
          if constexpr (kSplit) {
            // split-KV: the normalised partial output stays fp32 for the merge
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(part_row + col)[i] =
                  make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                              __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
          } else {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
              w[i] = pack2(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv, a.is_bf16);
            // whole 32-byte sectors per store: a lane's row is 1 KB away from its neighbour's
            if (hg < n1) {
              ptx::st_global_v8(out_row + col * 2, w);
              ptx::st_global_v8(out_row + col * 2 + 32, w + 8);
            }
          }
        }
        ptx::tc_fence_before();
        signal_lead(o_free, o_free_lead);
        SFA_PROF(6);
        if (half == 0) {
          // max of the scaled scores and sum of exp(score - max), back from the log2 domain
          if constexpr (kSplit) {
            a.part_m[(int64_t)item * kSfaHeads + hg] = m_true * 0.6931471805599453f;
            a.part_l[(int64_t)item * kSfaHeads + hg] = l_tot * ex2(m_ref - m_true);
          } else if (a.p.return_lse && hg < n1) {
            a.p.softmax_max[(int64_t)row * n1 + hg] = m_true * 0.6931471805599453f;
            a.p.softmax_sum[(int64_t)row * n1 + hg] = l_tot * ex2(m_ref - m_true);
          }
        }
      }
      SFA_PROF_STORE(4, threadIdx.x == kSfaSoftWarp0 * 32);
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies / MMAs in flight land
  }
  ptx::tc_fence_before();
  __syncthreads();
  // neither CTA may leave while its peer can still signal it or run a pair MMA on its memory
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == kSfaQkWarp0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(a.status, misaligned ? 2 : 1);
}

// ---- host side ---------------------------------------------------------------------------------
inline bool sfa_sm100_eligible(const DsaSfaParams* p) {
  // fewer than 128 heads (a tensor-parallel shard) run with the spare rows carrying zero queries;
  // below 16 heads the portable kernel wastes less
  if (p->n1 < 16 || p->n1 > kSfaHeads || p->d != 512 || p->d_rope != 64) return false;
  if ((int64_t)p->sparse_count * p->sparse_block_size > kSfaMaxSlots) return false;
  if (((uintptr_t)p->query & 15u) || ((uintptr_t)p->query_rope & 15u) || ((uintptr_t)p->key & 15u) ||
      ((uintptr_t)p->key_rope & 15u) || ((uintptr_t)p->out & 31u))
    return false;
  if (p->key_rows < 1 || p->key_rows >= (1ll << 31) - 1) return false;
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
  for (int32_t e = threadIdx.x; e < 8 * (kSfaDv / 4); e += 256) {
    const int32_t h = blockIdx.y * 8 + e / (kSfaDv / 4), c4 = e % (kSfaDv / 4);
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
        const float4 o = reinterpret_cast<const float4*>(part_o + i * kSfaDv)[c4];
        acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
        den += w;
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    uint2 packed;
    packed.x = pack2(acc.x * inv, acc.y * inv, is_bf16);
    packed.y = pack2(acc.z * inv, acc.w * inv, is_bf16);
    reinterpret_cast<uint2*>((unsigned char*)p.out + ((int64_t)row * p.n1 + h) * kSfaDv * 2)[c4] = packed;
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
  w.total = w.part_o + (split > 1 ? (size_t)rows * split * kSfaHeads * kSfaDv * 4 : 0);
  return w;
}
inline size_t sfa_sm100_workspace_bytes(const DsaSfaParams* p) {
  const int64_t rows = p->layout_q == DSA_LAYOUT_TND ? p->s1 : (int64_t)p->batch * p->s1;
  const int64_t slots = (int64_t)p->sparse_count * p->sparse_block_size;
  return sfa_sm100_ws_layout(rows, slots).total;
}

// SM count of a device, queried once per device; the first call on a device also raises the
// kernels' shared-memory limit there.  Safe to call from several host threads.
inline int sfa_sm100_device_sms(int dev) {
  static std::atomic<int> sm_count[64];
  static std::mutex setup_lock;
  if (dev < 0 || dev >= 64) return 0;
  int n = sm_count[dev].load(std::memory_order_acquire);
  if (n > 0) return n;
  std::lock_guard<std::mutex> g(setup_lock);
  n = sm_count[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 2) return 0;
  // the in-kernel register hand-over is sized for kSfaLaunchRegs registers per thread at launch: a
  // build that allocates a different number must not run (setmaxnreg.inc could block for good)
  cudaFuncAttributes fa0, fa1;
  if (cudaFuncGetAttributes(&fa0, sfa_fwd_sm100_kernel<false>) != cudaSuccess ||
      cudaFuncGetAttributes(&fa1, sfa_fwd_sm100_kernel<true>) != cudaSuccess ||
      fa0.numRegs != kSfaLaunchRegs || fa1.numRegs != kSfaLaunchRegs)
    return 0;
  if (cudaFuncSetAttribute(sfa_fwd_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)kSfaSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(sfa_fwd_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)kSfaSmemBytes) != cudaSuccess)
    return 0;
  sm_count[dev].store(n, std::memory_order_release);
  return n;
}

inline int sfa_sm100_launch(const DsaSfaParams* p, const SfaDev& d, int32_t* status, void* scratch, cudaStream_t st) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return DSA_ERR_CUDA;
  const int sms = sfa_sm100_device_sms(dev);
  if (sms < 2) return DSA_ERR_CUDA;
  const bool bf16 = p->dtype == DSA_DTYPE_BF16;
  const int64_t slots = (int64_t)p->sparse_count * p->sparse_block_size;
  const SfaWsLayout w = sfa_sm100_ws_layout(d.rows, slots);
  const int32_t split = sfa_sm100_split(d.rows, slots);
  const int32_t part_keys = split > 1 ? sfa_sm100_part_keys(slots, split) : (int32_t)((slots + kSfaBK - 1) / kSfaBK) * kSfaBK;
  int2* nvalid = reinterpret_cast<int2*>((char*)scratch + w.nvalid);
  int32_t* key_list = reinterpret_cast<int32_t*>((char*)scratch + w.key_list);
  sfa_compact_kernel<<<(d.rows + 3) / 4, 128, 0, st>>>(d, nvalid, key_list, split, part_keys, (int32_t)p->key_rows);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  SfaSm100Args a;
  a.p = d;
  a.status = status;
  a.idesc_qk = ptx::idesc_f16(bf16 ? 1u : 0u, 128, kSfaBK, 0, 0);
  a.idesc_pv = ptx::idesc_f16(bf16 ? 1u : 0u, 128, 256, 0, 1);
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.is_bf16 = bf16 ? 1 : 0;
  a.nvalid = nvalid;
  a.key_list = key_list;
  a.split = split;
  a.part_keys = part_keys;
  a.items = d.rows * split;
  a.part_m = reinterpret_cast<float*>((char*)scratch + w.part_m);
  a.part_l = reinterpret_cast<float*>((char*)scratch + w.part_l);
  a.part_o = reinterpret_cast<float*>((char*)scratch + w.part_o);
  int clusters = sms / 2;
#ifdef DSA_SFA_MAX_CLUSTERS
  clusters = DSA_SFA_MAX_CLUSTERS;
#endif
  if (clusters > a.items) clusters = a.items;
  CUtensorMap tkn, tkr, tq, tqr;
  if (!make_tmap_gather4_16bit(&tkn, p->key, (uint64_t)p->key_rows, 512, 1024, 64, bf16)) return DSA_ERR_CUDA;
  if (!make_tmap_gather4_16bit(&tkr, p->key_rope, (uint64_t)p->key_rows, 64, 128, 64, bf16)) return DSA_ERR_CUDA;
  if (!make_tmap_3d_16bit(&tq, p->query, (uint64_t)d.rows, (uint64_t)p->n1, 512, 1024, (uint64_t)p->n1 * 1024,
                          kSfaCtaHeads, 64, bf16))
    return DSA_ERR_CUDA;
  if (!make_tmap_3d_16bit(&tqr, p->query_rope, (uint64_t)d.rows, (uint64_t)p->n1, 64, 128, (uint64_t)p->n1 * 128,
                          kSfaCtaHeads, 64, bf16))
    return DSA_ERR_CUDA;
  if (split > 1) sfa_fwd_sm100_kernel<true><<<clusters * 2, kSfaThreads, kSfaSmemBytes, st>>>(tkn, tkr, tq, tqr, a);
  else sfa_fwd_sm100_kernel<false><<<clusters * 2, kSfaThreads, kSfaSmemBytes, st>>>(tkn, tkr, tq, tqr, a);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  if (split > 1) {
    sfa_merge_kernel<<<dim3(d.rows, kSfaHeads / 8), 256, 0, st>>>(d, split, a.part_o, a.part_m, a.part_l, a.is_bf16);
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  }
  return DSA_OK;
}

}  // namespace dsa
