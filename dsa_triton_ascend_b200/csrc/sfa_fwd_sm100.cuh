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
// hardware shares between the two tensor cores.  That fixes what each CTA needs per 64-key tile:
//   S tile  [128 heads x 64 keys]  : B = K rows, split along the keys  -> CTA c needs 32 of the
//                                    tile's 64 keys with all 576 features  (36 KB, K-major)
//   O       [128 heads x 512 cols] : B = V rows, split along the value columns -> CTA c needs
//                                    all 64 keys, columns {c*128.., 256+c*128..} (32 KB, MN-major)
// (two N = 256 MMAs per 16-key step: the first produces value columns 0..255, the second
// 256..511).  The two operand blocks of a CTA cannot alias: a pair MMA reads both CTAs at the SAME
// shared-memory offsets, the score product needs identical features at an offset and the value
// product identical keys.
//
// Data movement.  Only the K block is gathered from L2: TMA tile::gather4 loads into the
// 128-byte-swizzled MMA layout, issued by six producer warps from a front-packed list of physical
// KV rows that a pre-pass kernel writes.  The SM's TMA unit is the scarce resource here (it
// saturates at one 512-byte gather4 per ~18 cycles, bulk copies included), so the V block is not
// gathered a second time: four copier warps build it from the K block, which already holds this
// CTA's 32 keys with all columns - plain loads / stores for the columns this CTA owns, st.async
// into the peer's shared memory for the columns the peer owns.
//
// Accumulator layout of a pair MMA with M = 128 (measured): lanes 0..63 hold a CTA's rows with the
// first half of N, lanes 64..127 the same rows with the second half.  So TMEM lane L of CTA c
// belongs to head 64c + (L & 63); for S it holds the tile's keys 32*(L>>6) .. +31, for O the value
// columns j*256 + 128*(L>>6) .. +127 of MMA j.
//
// Softmax.  Two groups of four warps take alternate tiles (group g: S buffer g, P buffer g), so one
// tile's exponentials overlap the other's tensor-memory reads, barrier waits and P stores.  The
// probabilities of a row are scaled by ONE reference maximum, that of the row's first tile (its two
// halves exchanged through shared memory once per token): later tiles neither exchange anything
// nor wait for the tile before them, and O is never rescaled.  P may then exceed 1; a row whose
// later scores exceed the reference by more than a guard (2^60 for bf16, 2^12 for fp16: P and the
// fp32 sums stay finite) is marked and recomputed afterwards by the portable kernel
// (sfa_redo_kernel), which is exact for any input.  The true maximum and the row sum, which the
// softmax statistics need, are kept per thread and combined at the end of the token.
//
// Tensor memory per CTA: O 0..255 | S partials (2 buffers x 3 issuers x 32 columns) 256..447.
// Shared memory per CTA: Q_c 72 KB (A operand, loaded per token by TMA) | 2 x 36 KB K slots |
// 2 x 32 KB V slots | 2 x 8 KB P (A operand of the value product) | 2.5 KB exchange buffers.
//
// Warps (768 threads): 0..5 K gather producers, 6 Q loader, 8..10 QK^T issuers (issuer i owns
// feature blocks 3i..3i+2 and a partial S: one thread issues a short N = 64 MMA only every 60-90
// cycles), 11 PV issuer, 12..15 V copiers, 16..19 / 20..23 softmax groups.  MMAs are issued by the
// even CTA only; in the odd CTA the issuer warps relay "my operand has landed" to the even CTA's
// barriers instead.  All waits are bounded; a wait that gives up sets the status word.
#pragma once

#include <algorithm>
#include <atomic>
#include <mutex>

#include "ptx_sm100.cuh"
#include "sfa_fwd_mma.cuh"

namespace dsa {

constexpr int kSfaHeads = 128;       // heads per CTA pair
constexpr int kSfaCtaHeads = 64;
constexpr int kSfaBK = 64;           // keys per tile
constexpr int kSfaHalfBK = 32;       // keys of a tile each CTA gathers for the score product
constexpr int kSfaThreads = 768;
constexpr int kSfaQkLanes = 3;       // QK^T issuers
constexpr int kSfaKWarps = 6;        // warps 0..5: two per issuer
constexpr int kSfaQWarp = 6;         // Q loader (warp 7 idle)
constexpr int kSfaQkWarp0 = 8;       // warps 8..10
constexpr int kSfaPvWarp = 11;
constexpr int kSfaCopyWarp0 = 12;    // warps 12..15
constexpr int kSfaSoftWarp0 = 16;    // warps 16..19 (group 0), 20..23 (group 1)
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
constexpr uint32_t kSfaOffX = kSfaOffP + 2 * kSfaPBuf;       // float xm[2][128] | float mref[64] (+ pad) | float2 fin[2][64]
constexpr uint32_t kSfaOffBar = kSfaOffX + 1024 + 512 + 1024;
constexpr uint32_t kSfaSmemBytes = kSfaOffBar + 512;
static_assert(kSfaOffK % 1024 == 0 && kSfaOffV % 1024 == 0 && kSfaOffP % 1024 == 0, "operand alignment");
static_assert(kSfaSmemBytes <= 232448, "shared memory");

// setmaxnreg.inc only ever gets registers that warps of the SAME CTA have released and blocks (for
// good) until it has them: what the softmax warps ask for must fit into what the others give back.
constexpr int kSfaLaunchRegs = 80;   // 65536 / 768 threads, rounded down to a multiple of 8
constexpr int kSfaRegsLow = 56;      // warps 0..11
constexpr int kSfaRegsCopy = 104;    // warps 12..15 (a tile's 16 chunks of 16 bytes sit in registers)
constexpr int kSfaRegsHigh = 104;    // warps 16..23
static_assert((kSfaRegsHigh - kSfaLaunchRegs) * (kSfaThreads / 32 - kSfaSoftWarp0) +
                      (kSfaRegsCopy - kSfaLaunchRegs) * (kSfaSoftWarp0 - kSfaCopyWarp0) <=
                  (kSfaLaunchRegs - kSfaRegsLow) * kSfaCopyWarp0,
              "setmaxnreg: more registers requested than released");
static_assert(kSfaLaunchRegs * kSfaThreads <= 65536, "register file");

constexpr uint32_t kTmO = 0, kTmS = 256;
// The reference maximum of a row is fixed by its first tile; a later score may exceed it by this many
// log2 units before the row is handed to the portable kernel (P must stay finite in the io dtype and
// the fp32 sums of up to 8192 of them far from overflow).
constexpr float kSfaGuardBf16 = 60.f, kSfaGuardFp16 = 12.f;

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
  // rows whose scores outgrew the guard: flag per row (set once), list and count for sfa_redo_kernel
  int32_t* redo;            // [rows]
  int32_t* redo_list;       // [rows]
  int32_t* redo_count;      // [1]
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
// slot order, and their count.  A slot whose paged block is absent inside the valid length takes
// part as a zero row, like the reference's un-paged cache
// (sparse_flash_attention_triton.py:1012-1033): it gets the row number `oob_row` (= the number of
// KV rows), which the gather loads as zeros.
__global__ void __launch_bounds__(128) sfa_compact_kernel(SfaDev p, int2* __restrict__ nvalid,
                                                          int32_t* __restrict__ key_list, int32_t split,
                                                          int32_t part_keys, int32_t oob_row,
                                                          int32_t* __restrict__ redo,
                                                          int32_t* __restrict__ redo_count,
                                                          int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int32_t row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (blockIdx.x == 0 && threadIdx.x == 0) *redo_count = 0;
  // the workspace header (status word of the call) starts at zero: cleared here instead of by a
  // memset node of its own in front of the operator's launches
  if (blockIdx.x == 0 && threadIdx.x < 64) status[threadIdx.x] = 0;
  if (row >= p.rows) return;
  if (lane == 0) redo[row] = 0;
  const RowInfo ri = row_info(p.seq, row);
  const int32_t slots = p.sparse_count * p.sparse_block_size;
  const int32_t* idx_row = p.sparse_indices + (int64_t)row * p.sparse_count;
  int32_t* out = key_list + (int64_t)row * slots;
  int32_t n = 0;
  if (ri.pos < ri.act_q && ri.threshold > 0 && ri.act_k > 0) {
    // token-wise indices whose rows start on 16-byte boundaries: four slots per lane and step (one
    // 16-byte load; slot order = lane-major, so a lane's place is the valid slots of the lanes below
    // it plus its own earlier ones)
    const bool wide = p.sparse_block_size == 1 && (p.sparse_count & 3) == 0 &&
                      ((reinterpret_cast<uintptr_t>(p.sparse_indices) & 15) == 0);
    // (four steps are resolved together so that their index loads and block-table look-ups are in
    // flight at the same time: with few rows - decode - the pre-pass is bound by that latency)
    for (int32_t j0 = 0; wide && j0 < slots; j0 += 512) {
      int4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int32_t j = j0 + u * 128 + 4 * lane;
        v[u] = make_int4(-1, -1, -1, -1);
        if (j < slots) v[u] = *reinterpret_cast<const int4*>(idx_row + j);
      }
      int32_t prow[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int32_t id[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int64_t r = -1;
          const int64_t tok = id[e];
          if (tok >= 0 && tok < ri.threshold && tok < ri.act_k &&
              (p.seq.layout_k == DSA_LAYOUT_PA_BSND || tok < p.seq.s2)) {
            r = key_row(p.seq, ri, (int32_t)tok);
            if (r < 0 || r >= oob_row) r = oob_row;
          }
          prow[u][e] = (int32_t)r;
        }
      }
      const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t below = 0, total = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t m = __ballot_sync(0xffffffffu, prow[u][e] >= 0);
          below += __popc(m & lt);
          total += __popc(m);
        }
        int32_t* o = out + n + below;
        if (total == 128 && ((n & 3) == 0)) {
          *reinterpret_cast<int4*>(o) = make_int4(prow[u][0], prow[u][1], prow[u][2], prow[u][3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (prow[u][e] >= 0) *o++ = prow[u][e];
        }
        n += (int32_t)total;
      }
    }
    for (int32_t j0 = wide ? slots : 0; j0 < slots; j0 += 32) {
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
  float* xm = reinterpret_cast<float*>(sfa_sm + kSfaOffX);     // [2 groups][128] exchange between the halves of a head
  float* mref = xm + 256;                                       // [64] the token's reference maximum per head (from its first tile)
  float2* fin = reinterpret_cast<float2*>(xm + 256 + 128);      // [2 groups][64] (row sum, true maximum) of a group at the end of a token
  uint64_t* bars = reinterpret_cast<uint64_t*>(sfa_sm + kSfaOffBar);
  // K barriers are indexed [slot * 3 + issuer]: every issuer's three feature blocks are handed over
  // and released on their own.
  uint64_t* k_full = bars;         // [6] gather -> QK issuer / relay, copiers              (tx bytes)
  uint64_t* k_empty = bars + 6;    // [6] blocks read by the issuer's MMAs (commit) and by the four copier warps -> K producers
  uint64_t* k_ready = bars + 12;   // [6] even CTA only: the odd CTA's blocks have landed
  uint64_t* v_full = bars + 18;    // [2] own copier warps (4 arrivals + 1 arming) and the peer's st.async bytes -> PV issuer / relay
  uint64_t* v_empty = bars + 20;   // [2] PV of the tile done -> copiers                     (commit, both CTAs)
  uint64_t* v_ready = bars + 22;   // [2] even CTA only: the odd CTA's V slot is complete
  uint64_t* s_full = bars + 24;    // [2] all three partial products done -> softmax group   (commit x 3, both CTAs)
  uint64_t* s_empty = bars + 26;   // [2] even CTA only: the group's warps of both CTAs hold S in registers
  uint64_t* p_full = bars + 28;    // [2] even CTA only: P stored in both CTAs
  uint64_t* p_empty = bars + 30;   // [2] PV done -> softmax                                 (commit, both CTAs)
  uint64_t* q_full = bars + 32;    // this CTA's Q has landed (tx bytes)
  uint64_t* q_ready = bars + 33;   // even CTA only: the odd CTA's Q has landed
  uint64_t* q_empty = bars + 34;   // all QK issuers are through with the token              (commit x 3, both CTAs)
  uint64_t* o_free = bars + 35;    // even CTA only: epilogue warps of both CTAs have read O
  // The two halves of a head sit in warps q and q + 2 of a group ("pair" q & 1): exchanges between
  // them (first tile of a token, end of a token) only involve that pair.
  uint64_t* x_bar = bars + 36;     // [group * 2 + pair] xm written (2 warps)
  uint64_t* xr_bar = bars + 40;    // [group * 2 + pair] xm read, it may be written again (2 warps)
  uint64_t* m_bar = bars + 44;     // [pair] mref written for the token (the 2 warps of the pair in the group of its first tile)
  uint64_t* e_bar = bars + 48;     // both groups: fin written
  uint64_t* er_bar = bars + 49;    // both groups: fin read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 50);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 51);
  static_assert(52 * 8 <= 512, "barrier area");

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
    for (int i = 0; i < 4; ++i) {
      ptx::mbar_init(&x_bar[i], 2); ptx::mbar_init(&xr_bar[i], 2);
    }
    for (int i = 0; i < 2; ++i) ptx::mbar_init(&m_bar[i], 2);
    ptx::mbar_init(q_full, 1);
    ptx::mbar_init(q_ready, 1);
    ptx::mbar_init(q_empty, kSfaQkLanes);
    ptx::mbar_init(o_free, 16);
    ptx::mbar_init(e_bar, 8);
    ptx::mbar_init(er_bar, 8);
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

  // Registers: kSfaLaunchRegs per thread at launch; producers and issuers give some back, the
  // copier and softmax warps take them (whole warpgroups of four warps change together).  Each
  // class of roles sits in its own branch, right under its setmaxnreg: the compiler budgets a
  // branch by the setmaxnreg that dominates it.
  if (warp < kSfaCopyWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kSfaRegsLow));
    if (*abort_flag) {
      // nothing started: fall through to the teardown
    } else if (warp < kSfaKWarps) {
      // ------------------------------------------------------------------ K gather producers
      // Two warps per QK^T issuer: 8 row groups (4 of this CTA's 32 keys each) x the issuer's 3
      // column blocks = 24 gather4 loads of 512 bytes per tile, dealt out over the two warps.  The
      // lanes of a warp issue one after the other (~100 cycles per load), warps issue in parallel
      // until the SM's TMA unit saturates at one load per ~18 cycles.
      const int qi = warp >> 1;                          // the issuer this warp feeds
      const int gw = warp & 1;
      const int o = gw + 2 * lane;
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
      // (the four keys of a load are consecutive entries of the list: one 16-byte load when the
      // row's list starts on a 16-byte boundary, except in a row's last tile, where keys past the
      // end re-read the tile's first key and are masked by the softmax)
      auto load_rows = [&](const TilePos& tp, int32_t* r) {
        if (!active || tp.item >= a.items) { r[0] = r[1] = r[2] = r[3] = 0; return; }
        const int32_t* list = a.key_list + tp.off + tp.t * kSfaBK;
        if ((tp.t + 1) * kSfaBK <= tp.nvalid && (tp.off & 3) == 0) {
          const int4 v = *reinterpret_cast<const int4*>(list + key0);
          r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
        } else {
          const int32_t left = tp.nvalid - tp.t * kSfaBK;
#pragma unroll
          for (int i = 0; i < 4; ++i) r[i] = list[key0 + i < left ? key0 + i : 0];
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
        // every lane polls (see ptx::mbar_wait_warp): the gather below is issued for the lanes one
        // after the other and must find the warp converged.  Like every wait of this kernel it
        // spins without suspending: waking from a suspended try_wait costs hundreds of cycles at
        // every hand-over (826 vs 640 TFLOP/s on a 4096-token, top-2048 case).
        ok = ptx::mbar_spin_warp(&empty[s * 3], (use & 1) ^ 1, abort_flag);
        if (!ok) break;
        SFA_PROF(1);
        if (gw == 0 && lane == 0) ptx::mbar_arrive_expect_tx(&full[s * 3], kSfaKSub);
        __syncwarp();
        if (active) {
          if (blk == 8) ptx::tma_gather4_2d(slot0 + s * kSfaKSlot, &tmap_kr, &full[s * 3], 0, rc[0], rc[1], rc[2], rc[3]);
          else ptx::tma_gather4_2d(slot0 + s * kSfaKSlot, &tmap_kn, &full[s * 3], x, rc[0], rc[1], rc[2], rc[3]);
        }
        __syncwarp();
        SFA_PROF(2);
        ++n_tile;
        cur = nxt;
#pragma unroll
        for (int i = 0; i < 4; ++i) rc[i] = rn[i];
      }
      SFA_PROF_STORE(0, lane == 0 && warp == 0);
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
      // softmax adds the three partials.  The loop is warp-uniform (every lane waits) and only the
      // MMAs and the commits are issued by one elected lane.
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
          ok = ptx::mbar_spin_warp(q_full, n_tok & 1, abort_flag) && ptx::mbar_spin_cluster_warp(q_ready, n_tok & 1, abort_flag);
        }
        SFA_PROF(5);
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          const uint32_t b = n_tile & 1, use = n_tile >> 1, kb = b * kSfaQkLanes + qi;
          SFA_PROF(0);
          ok = ptx::mbar_spin_warp(&k_full[kb], use & 1, abort_flag);
          if (!ok) break;
          SFA_PROF(1);
          if (rank != 0) {
            // relaxed: the blocks were written by the TMA unit and are complete once the barrier
            // says so; nothing of this thread's own has to be published
            if (ptx::elect_one()) ptx::mbar_arrive_remote_relaxed(k_ready_lead + kb * 8, 0u);
            __syncwarp();
            continue;
          }
          ok = ptx::mbar_spin_cluster_warp(&k_ready[kb], use & 1, abort_flag);
          SFA_PROF(2);
          ok = ok && ptx::mbar_spin_cluster_warp(&s_empty[b], (use & 1) ^ 1, abort_flag);
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
        if (rank == 0) ok = ptx::mbar_spin_cluster_warp(o_free, (n_tok & 1) ^ 1, abort_flag);
        SFA_PROF(5);
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          const uint32_t b = n_tile & 1, use = n_tile >> 1;
          SFA_PROF(0);
          ok = ptx::mbar_spin_cluster_warp(&v_full[b], use & 1, abort_flag);
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
          ok = ptx::mbar_spin_cluster_warp(&v_ready[b], use & 1, abort_flag);
          SFA_PROF(2);
          ok = ok && ptx::mbar_spin_cluster_warp(&p_full[b], use & 1, abort_flag);
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
  } else if (warp < kSfaSoftWarp0) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSfaRegsCopy));
    if (!*abort_flag) {
      // ------------------------------------------------------------------ V copiers
      // These 128 threads copy the four column blocks of the K slot that this CTA owns as value
      // columns into its own V slot (plain loads and stores) and the four that the peer owns into
      // the peer's V slot (st.async: the bytes are counted on the peer's barrier when they land,
      // the sender does not wait), rows 32*rank.. of every block; 16 chunks of 16 bytes per thread.
      // Byte offsets inside 4 KB are kept, so the 128-byte swizzle pattern carries over.
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
          ok = ptx::mbar_spin_warp(&k_full[b * 3], use & 1, abort_flag) &&
               ptx::mbar_spin_warp(&k_full[b * 3 + 1], use & 1, abort_flag) &&
               ptx::mbar_spin_warp(&k_full[b * 3 + 2], use & 1, abort_flag);
          if (!ok) break;
          SFA_PROF(1);
          // The tile's 16 chunks go into registers first and the K slot is handed back at once: its
          // refill must not wait for the V slot, which is only free when the value product two
          // tiles back has completed (the registers act as a third V stage).
          const unsigned char* ksrc = k_s + b * kSfaKSlot;
          uint4 v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // i < 8: the four blocks this CTA owns (local copy), i >= 8: the four the peer owns (remote)
            const int owner = i < 8 ? (int)rank : (int)peer;
            const int q = (i & 7) * 128 + tid;                  // 0..1023: chunk within the four blocks
            const int pblk = q >> 8, within = q & 255;
            const int fblk = 4 * (pblk >> 1) + 2 * owner + (pblk & 1);
            v[i] = *reinterpret_cast<const uint4*>(ksrc + fblk * kSfaKBlk + within * 16);
          }
          // The slot goes back to the TMA unit: reads through the generic proxy (the loads above)
          // and the writes of the next gather through the async proxy are only ordered by a proxy
          // fence.  Without it the gather was seen to overtake these loads (outputs changed from
          // run to run once the hand-overs of this kernel got fast).
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane < 3) ptx::mbar_arrive(&k_empty[b * 3 + lane]);
          SFA_PROF(2);
          // V slot b is free in both CTAs once the product that read it has completed
          ok = ptx::mbar_spin_warp(&v_empty[b], (use & 1) ^ 1, abort_flag);
          if (!ok) break;
          SFA_PROF(3);
          // the peer's half of my V slot: 16 KB of transaction bytes
          if (tid == 0) ptx::mbar_arrive_expect_tx(&v_full[b], kSfaVSlot / 2);
          const uint32_t vdst = b * kSfaVSlot + rank * kSfaKBlk;     // rows 32*rank.. of a V block
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int q = (i & 7) * 128 + tid;
            const int pblk = q >> 8, within = q & 255;
            const uint32_t off = vdst + pblk * kSfaVBlk + within * 16;
            if (i >= 8) ptx::st_async_v4(v_peer + off, v[i], v_full_peer + b * 8);
            else *reinterpret_cast<uint4*>(v_s + off) = v[i];
          }
          // the local rows are made visible to the tensor core's reads before the arrival says so
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&v_full[b]);
          SFA_PROF(4);
        }
      }
      SFA_PROF_STORE(1, tid == 0);
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSfaRegsHigh));
    if (!*abort_flag) {
      // ------------------------------------------------------------------ softmax + epilogue
      const int g = (warp - kSfaSoftWarp0) >> 2;    // group: takes the tiles with (tile number & 1) == g
      const int quarter = warp & 3;
      const int L = quarter * 32 + lane;            // TMEM lane
      const int hl = L & 63, half = L >> 6;         // head within this CTA; which half of N this lane holds
      const int32_t hg = (int32_t)rank * kSfaCtaHeads + hl;
      const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
      const uint32_t s_empty_lead = ptx::map_to_rank(&s_empty[g], 0);
      const uint32_t p_full_lead = ptx::map_to_rank(&p_full[g], 0);
      const uint32_t o_free_lead = ptx::map_to_rank(o_free, 0);
      float* xmg = xm + g * 128;
      const int gp = g * 2 + (quarter & 1);         // this warp's pair
      const float guard = a.is_bf16 ? kSfaGuardBf16 : kSfaGuardFp16;
      uint32_t n_tile = 0, n_tok = 0, n_x = 0;
      bool ok = true;
      SFA_PROF_DECL;
      // waits are warp-wide: the tcgen05 loads / stores that follow are warp-collective and must
      // never run with part of a warp gone
      auto wait_w = [&](uint64_t* bar, uint32_t parity) -> bool { return ptx::mbar_spin_warp(bar, parity, abort_flag); };
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
      // Value of the head's other thread in this group (lane L ^ 64, another warp) through shared
      // memory.  The buffer is written again only after everybody has read it (xr_bar).
      auto exchange = [&](float v, float& other) -> bool {
        bool got = n_x == 0 || ptx::mbar_spin_warp(&xr_bar[gp], (n_x - 1) & 1, abort_flag);
        xmg[L] = v;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&x_bar[gp]);
        got = ptx::mbar_spin_warp(&x_bar[gp], n_x & 1, abort_flag) && got;
        other = xmg[L ^ 64];
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&xr_bar[gp]);
        ++n_x;
        return got;
      };
      for (int32_t item = cluster_id; item < a.items && ok; item += n_clusters) {
        const int32_t nvalid = a.nvalid[item].x;
        const int32_t ntiles = (nvalid + kSfaBK - 1) / kSfaBK;
        const int32_t row = kSplit ? item / a.split : item;
        // this lane's output columns: group g stores the columns of MMA j = g, g * 256 + half * 128 + 0..127
        const int col0 = g * 256 + half * 128;
        unsigned char* out_row = (unsigned char*)a.p.out + (((int64_t)row * n1 + hg) * kSfaDv + col0) * 2;
        float* part_row = kSplit ? a.part_o + ((int64_t)item * kSfaHeads + hg) * kSfaDv + col0 : nullptr;
        if (ntiles == 0) {
          if constexpr (kSplit) {
            // an empty part: the merge skips it
            if (g == 0 && half == 0) { a.part_m[(int64_t)item * kSfaHeads + hg] = 0.f; a.part_l[(int64_t)item * kSfaHeads + hg] = 0.f; }
          } else if (hg < n1) {
            // nothing visible: zeros in all three outputs
#pragma unroll
            for (int c = 0; c < 16; ++c) reinterpret_cast<uint4*>(out_row)[c] = make_uint4(0, 0, 0, 0);
            if (g == 0 && half == 0 && a.p.return_lse) {
              a.p.softmax_max[(int64_t)row * n1 + hg] = 0.f;
              a.p.softmax_sum[(int64_t)row * n1 + hg] = 0.f;
            }
          }
          continue;
        }
        // This thread's share of the row sum, relative to the token's reference maximum m_ref = the
        // maximum of the row's FIRST tile.  Later tiles use it as it is: nothing is exchanged per
        // tile and no tile waits for the one before it; O is never rescaled.  P = 2^(s - m_ref) may
        // exceed 1, which the io dtype and the fp32 sums hold up to the guard; a row that outgrows it
        // is recomputed by the portable kernel afterwards (sfa_redo_kernel).
        float m_ref = 0.f, mt = -INFINITY, l = 0.f, l_grp = 0.f;
        bool have_ref = false, outgrown = false;
        for (int32_t t = 0; t < ntiles && ok; ++t, ++n_tile) {
          if ((int)(n_tile & 1u) != g) continue;
          const uint32_t use = n_tile >> 1;
          const int32_t cnt = min(kSfaBK, nvalid - t * kSfaBK) - half * kSfaHalfBK;   // valid keys among this lane's 32
          SFA_PROF(7);
          ok = wait_w(&s_full[g], use & 1);
          if (!ok) break;
          SFA_PROF(0);
          ptx::tc_fence_after();
          float sc[kSfaHalfBK];
          {
            // the three issuers' partial products
            float s1[kSfaHalfBK];
            ptx::tmem_ld_x32(lane_addr + kTmS + (g * kSfaQkLanes) * 32, reinterpret_cast<uint32_t*>(sc));
            ptx::tmem_ld_x32(lane_addr + kTmS + (g * kSfaQkLanes + 1) * 32, reinterpret_cast<uint32_t*>(s1));
            ptx::tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < kSfaHalfBK; ++k) sc[k] += s1[k];
            ptx::tmem_ld_x32(lane_addr + kTmS + (g * kSfaQkLanes + 2) * 32, reinterpret_cast<uint32_t*>(s1));
            ptx::tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < kSfaHalfBK; ++k) sc[k] += s1[k];
          }
          ptx::tc_fence_before();
          signal_lead(&s_empty[g], s_empty_lead);
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
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          mt = fmaxf(mt, mx);
          SFA_PROF(2);
          if (t == 0) {
            // the row's first tile fixes the reference: its maximum over both halves (the first half
            // always has a valid key), published for the other group
            float mx_other;
            ok = exchange(mx, mx_other);
            if (!ok) break;
            m_ref = fmaxf(mx, mx_other);
            // (everybody has read the previous token's entry: they arrive on er_bar after reading it)
            ok = n_tok == 0 || wait_w(er_bar, (n_tok - 1) & 1);
            if (!ok) break;
            if (half == 0) mref[hl] = m_ref;
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&m_bar[quarter & 1]);
            have_ref = true;
          } else if (!have_ref) {
            ok = wait_w(&m_bar[quarter & 1], n_tok & 1);
            if (!ok) break;
            m_ref = mref[hl];
            have_ref = true;
          }
          outgrown = outgrown || mx > m_ref + guard;
          SFA_PROF(3);
          float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int k = 0; k < kSfaHalfBK; k += 4) {
            sc[k] = ex2(sc[k] - m_ref); sc[k + 1] = ex2(sc[k + 1] - m_ref);
            sc[k + 2] = ex2(sc[k + 2] - m_ref); sc[k + 3] = ex2(sc[k + 3] - m_ref);
            sum4[0] += sc[k]; sum4[1] += sc[k + 1]; sum4[2] += sc[k + 2]; sum4[3] += sc[k + 3];
          }
          l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
          if (ntiles == 1) {
            // a single tile holds the whole row: normalise before rounding, as the golden does
            float l_other;
            ok = exchange(l, l_other);
            if (!ok) break;
            l_grp = l + l_other;
            const float inv = 1.f / l_grp;
#pragma unroll
            for (int k = 0; k < kSfaHalfBK; ++k) sc[k] *= inv;
          }
          // ---- P once the product that last read this P buffer has finished
          SFA_PROF(2);
          ok = wait_w(&p_empty[g], (use & 1) ^ 1);
          if (!ok) break;
          SFA_PROF(4);
          {
            // row hl of the K-major, 128-byte-swizzled A operand: keys half*32 .. +31 are the 16-byte
            // chunks half*4 .. +3 of the row
            unsigned char* prow = p_s + g * kSfaPBuf + hl * 128;
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
          signal_lead(&p_full[g], p_full_lead);
          SFA_PROF(5);
        }
        if (!ok) break;
        SFA_PROF(7);
        // ---- end of the token: row sum and true maximum over the four threads of the head (two
        // halves x two groups); a group without a tile contributes 0 / -inf
        const uint32_t last = n_tile - 1;
        float l_tot, mt_fin;
        {
          float l_other, mt_other;
          if (ntiles > 1) {
            ok = exchange(l, l_other);
            if (!ok) break;
            l_grp = l + l_other;
          } else if ((int)(last & 1u) != g) {
            l_grp = 0.f;                                   // (the tile's group normalised inside the tile)
          }
          ok = exchange(mt, mt_other);
          if (!ok) break;
          const float mt_grp = fmaxf(mt, mt_other);
          ok = n_tok == 0 || wait_w(er_bar, (n_tok - 1) & 1);
          if (!ok) break;
          if (half == 0) fin[g * 64 + hl] = make_float2(l_grp, mt_grp);
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(e_bar);
          ok = wait_w(e_bar, n_tok & 1);
          if (!ok) break;
          const float2 fo = fin[(g ^ 1) * 64 + hl];
          l_tot = l_grp + fo.x;
          mt_fin = fmaxf(mt_grp, fo.y);
          m_ref = mref[hl];                                // (a group without a tile has not read it yet)
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(er_bar);
        }
        if (outgrown && hg < n1 && atomicExch(&a.redo[row], 1) == 0) a.redo_list[atomicAdd(a.redo_count, 1)] = row;
        // ---- epilogue: wait for the last product, normalise, store this group's 128 columns
        ok = wait_w(&p_empty[last & 1], (last >> 1) & 1);
        if (!ok) break;
        ptx::tc_fence_after();
        const float inv = ntiles == 1 ? 1.f : 1.f / l_tot;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          // accumulator columns g*128 + c*32 .. +31 = value columns g*256 + half*128 + c*32 ..
          uint32_t o[32];
          ptx::tmem_ld_x32(lane_addr + kTmO + g * 128 + c * 32, o);
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
            // whole 32-byte sectors per store: a lane's row is 1 KB away from its neighbour's
            if (hg < n1) {
              ptx::st_global_v8(out_row + c * 64, w);
              ptx::st_global_v8(out_row + c * 64 + 32, w + 8);
            }
          }
        }
        ptx::tc_fence_before();
        signal_lead(o_free, o_free_lead);
        SFA_PROF(6);
        if (g == 0 && half == 0) {
          // max of the scaled scores and sum of exp(score - max), back from the log2 domain
          if constexpr (kSplit) {
            a.part_m[(int64_t)item * kSfaHeads + hg] = mt_fin * 0.6931471805599453f;
            a.part_l[(int64_t)item * kSfaHeads + hg] = l_tot * ex2(m_ref - mt_fin);
          } else if (a.p.return_lse && hg < n1) {
            a.p.softmax_max[(int64_t)row * n1 + hg] = mt_fin * 0.6931471805599453f;
            a.p.softmax_sum[(int64_t)row * n1 + hg] = l_tot * ex2(m_ref - mt_fin);
          }
        }
        ++n_tok;
      }
      SFA_PROF_STORE(4 + g, (warp & 3) == 0 && lane == 0);
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

// Workspace beyond the header: nvalid[rows * split], key_list[rows * slots], the redo flags, list
// and count, and for split > 1 the partial maxima, sums and outputs.
struct SfaWsLayout { size_t nvalid, key_list, redo, redo_list, redo_count, part_m, part_l, part_o, total; };
inline SfaWsLayout sfa_sm100_ws_layout(int64_t rows, int64_t slots) {
  const int32_t split = sfa_sm100_split(rows, slots);
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  SfaWsLayout w;
  w.nvalid = 0;
  w.key_list = up((size_t)rows * split * 8);
  w.redo = w.key_list + up((size_t)rows * slots * 4);
  w.redo_list = w.redo + up((size_t)rows * 4);
  w.redo_count = w.redo_list + up((size_t)rows * 4);
  w.part_m = w.redo_count + 256;
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
  const int redo_smem = (kSfaSimtHeads + kSfaSimtKeys) * (512 + 64 + kSfaSimtPad) * 2;
  if (cudaFuncSetAttribute(sfa_redo_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, redo_smem) !=
          cudaSuccess ||
      cudaFuncSetAttribute(sfa_redo_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, redo_smem) != cudaSuccess)
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
  int32_t* redo = reinterpret_cast<int32_t*>((char*)scratch + w.redo);
  int32_t* redo_list = reinterpret_cast<int32_t*>((char*)scratch + w.redo_list);
  int32_t* redo_count = reinterpret_cast<int32_t*>((char*)scratch + w.redo_count);
  sfa_compact_kernel<<<(d.rows + 3) / 4, 128, 0, st>>>(d, nvalid, key_list, split, part_keys, (int32_t)p->key_rows, redo,
                                                      redo_count, status);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  count_launch();
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
  a.redo = redo;
  a.redo_list = redo_list;
  a.redo_count = redo_count;
  int clusters = sms / 2;
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
  count_launch();
  if (split > 1) {
    sfa_merge_kernel<<<dim3(d.rows, kSfaHeads / 8), 256, 0, st>>>(d, split, a.part_o, a.part_m, a.part_l, a.is_bf16);
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
    count_launch();
  }
  {
    // rows whose scores outgrew the fixed reference maximum (normally none) are redone exactly
    const size_t smem = (size_t)(kSfaSimtHeads + kSfaSimtKeys) * (p->d + p->d_rope + kSfaSimtPad) * 2;
    const int64_t work = (int64_t)d.rows * ((p->n1 + kSfaSimtHeads - 1) / kSfaSimtHeads);
    const unsigned blocks = (unsigned)std::min<int64_t>(work, (int64_t)sms * 2);
    if (bf16) sfa_redo_kernel<__nv_bfloat16><<<blocks, kSfaSimtThreads, smem, st>>>(d, redo_list, redo_count);
    else sfa_redo_kernel<__half><<<blocks, kSfaSimtThreads, smem, st>>>(d, redo_list, redo_count);
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
    count_launch();
  }
  return DSA_OK;
}

}  // namespace dsa
