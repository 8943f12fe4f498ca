// C ABI of the library (declared in include/dsa_b200.h): argument validation, kernel choice,
// workspace layout and launches.  Host code only decides and enqueues; it never synchronises
// (except dsa_read_device_status) and never allocates device memory.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../../include/dsa_b200.h"
#include "dsa_common.cuh"
#include "li_score_simt.cuh"
#include "li_score_sm100.cuh"
#include "li_topk.cuh"
#include "sfa_fwd_mma.cuh"
#include "sfa_fwd_sm100.cuh"
#include "sfa_bwd_simt.cuh"
#include "sfa_bwd_mma.cuh"
#include "sli_grad.cuh"

namespace dsa {

constexpr size_t kWorkspaceHeader = 256;  // bytes reserved at the start of every workspace (status word)

static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

static int li_validate(const DsaLiParams* p) {
  if (p == nullptr) return DSA_ERR_NULL;
  if (p->struct_size != sizeof(DsaLiParams)) return DSA_ERR_STRUCT;
  if (!p->query || !p->key || !p->weights || !p->out_indices) return DSA_ERR_NULL;
  if (p->layout_q != DSA_LAYOUT_BSND && p->layout_q != DSA_LAYOUT_TND) return DSA_ERR_VALUE;
  if (p->layout_k < DSA_LAYOUT_BSND || p->layout_k > DSA_LAYOUT_PA_BSND) return DSA_ERR_VALUE;
  if (p->dtype_qk != DSA_DTYPE_BF16 && p->dtype_qk != DSA_DTYPE_FP16) return DSA_ERR_VALUE;
  if (p->dtype_w < DSA_DTYPE_BF16 || p->dtype_w > DSA_DTYPE_FP32) return DSA_ERR_VALUE;
  if (p->batch < 1 || p->s1 < 0 || p->s2 < 0 || p->n1 < 1 || p->n2 < 1 || p->d < 1) return DSA_ERR_VALUE;
  if (p->n1 % p->n2 != 0) return DSA_ERR_VALUE;  // lightning_indexer_triton.py:524-525
  if (p->d % 8 != 0) return DSA_ERR_VALUE;
  if (p->sparse_mode != 0 && p->sparse_mode != 3) return DSA_ERR_VALUE;
  if (p->rank_mode != DSA_RANK_IO_DTYPE && p->rank_mode != DSA_RANK_FP32) return DSA_ERR_VALUE;
  if (p->sparse_count < 1) return DSA_ERR_VALUE;
  if (p->sparse_count > kTopkMaxCount) return DSA_ERR_TOO_LARGE;
  if (p->s2 >= (1 << 24)) return DSA_ERR_TOO_LARGE;
  if (p->layout_q == DSA_LAYOUT_TND && (!p->seq_q || !p->seq_q_cumulative)) return DSA_ERR_VALUE;
  if (p->layout_k == DSA_LAYOUT_TND && (!p->seq_k || !p->seq_k_cumulative)) return DSA_ERR_VALUE;
  if (p->layout_k == DSA_LAYOUT_PA_BSND && (!p->block_table || p->block_size < 1 || p->max_blocks < 1 || !p->seq_k))
    return DSA_ERR_VALUE;
  // a paged sequence cannot be longer than its row of the block table (the score scratch and the
  // key tiles are sized from s2; positions past the table would never be written)
  if (p->layout_k == DSA_LAYOUT_PA_BSND && (int64_t)p->s2 > (int64_t)p->max_blocks * p->block_size) return DSA_ERR_VALUE;
  if (p->key_rows < 0) return DSA_ERR_VALUE;
  if (p->phases < 1 || p->phases > DSA_PHASE_ALL) return DSA_ERR_VALUE;
  if (p->kernel < DSA_KERNEL_AUTO || p->kernel > DSA_KERNEL_TENSOR) return DSA_ERR_VALUE;
  return DSA_OK;
}

static inline int64_t li_rows(const DsaLiParams* p) {
  return p->layout_q == DSA_LAYOUT_TND ? (int64_t)p->s1 : (int64_t)p->batch * p->s1;
}
static inline int64_t li_score_ld(const DsaLiParams* p) { return round_up(p->s2 > 0 ? p->s2 : 1, 4); }

static LiDev li_dev(const DsaLiParams* p) {
  LiDev d;
  d.seq.seq_q = p->seq_q; d.seq.seq_k = p->seq_k; d.seq.block_table = p->block_table;
  d.seq.layout_q = p->layout_q; d.seq.layout_k = p->layout_k;
  d.seq.seq_q_cum = p->seq_q_cumulative; d.seq.seq_k_cum = p->seq_k_cumulative;
  d.seq.batch = p->batch; d.seq.s1 = p->s1; d.seq.s2 = p->s2;
  d.seq.block_size = p->block_size; d.seq.max_blocks = p->max_blocks;
  d.seq.sparse_mode = p->sparse_mode;
  d.seq.key_rows = p->key_rows;
  d.query = p->query; d.key = p->key; d.weights = p->weights;
  d.out_indices = p->out_indices; d.out_values = p->out_values;
  d.dtype_w = p->dtype_w; d.n1 = p->n1; d.n2 = p->n2; d.d = p->d;
  d.rows = (int32_t)li_rows(p);
  d.sparse_count = p->sparse_count; d.rank_mode = p->rank_mode; d.return_value = p->return_value;
  return d;
}

// The tcgen05 score kernel serves the production shape; everything else runs on the portable one.
static bool li_takes_tensor_path(const DsaLiParams* p) {
  return p->kernel != DSA_KERNEL_PORTABLE && li_sm100_eligible(p);
}

template <typename T>
static int li_launch(const DsaLiParams* p, float* scores, cudaStream_t st, int32_t* status = nullptr) {
  LiDev d = li_dev(p);
  const int64_t ld = li_score_ld(p);
  const int64_t rown = (int64_t)d.rows * p->n2;
  if (rown == 0) return DSA_OK;
  if (p->phases & DSA_PHASE_SCORE) {
    if (p->s2 > 0 && status != nullptr && li_takes_tensor_path(p)) {
      int rc = li_sm100_launch(p, d, scores, ld, status, st);
      if (rc != DSA_OK) return rc;
    } else if (p->s2 > 0) {
      if ((p->s2 + kSimtKeys - 1) / kSimtKeys > 65535) return DSA_ERR_TOO_LARGE;   // key tiles ride on grid.y
      dim3 grid((unsigned)rown, (unsigned)((p->s2 + kSimtKeys - 1) / kSimtKeys), 1);
      li_score_simt_kernel<T><<<grid, kSimtKeys, 0, st>>>(d, scores, ld);
      if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
      count_launch();
    }
  }
  if (p->phases & DSA_PHASE_TOPK) {
    const bool rank16 = p->rank_mode == DSA_RANK_IO_DTYPE;
    if (p->s2 <= kTopkThreads * kTopkFastKeys && p->sparse_count <= kTopkThreads * 4) {
      // register / shuffle kernel: rows of up to 8192 keys, up to 2048 outputs
      const int e = p->sparse_count <= kTopkThreads ? 1 : (p->sparse_count <= 2 * kTopkThreads ? 2 : 4);
#define DSA_TOPK_FAST(R, E) li_topk_fast_kernel<T, R, E><<<(unsigned)rown, kTopkThreads, 0, st>>>(d, scores, ld)
      if (rank16) {
        // io-dtype ranking: one histogram on a linear scale selects and orders
        if (e == 1) li_topk_bins_kernel<T, 1><<<(unsigned)rown, kTopkThreads, 0, st>>>(d, scores, ld);
        else if (e == 2) li_topk_bins_kernel<T, 2><<<(unsigned)rown, kTopkThreads, 0, st>>>(d, scores, ld);
        else li_topk_bins_kernel<T, 4><<<(unsigned)rown, kTopkThreads, 0, st>>>(d, scores, ld);
      }
      else { if (e == 1) DSA_TOPK_FAST(false, 1); else if (e == 2) DSA_TOPK_FAST(false, 2); else DSA_TOPK_FAST(false, 4); }
#undef DSA_TOPK_FAST
    } else if (rank16 && p->sparse_count <= kTopkThreads * 4) {
      // longer rows, io-dtype ranking: the same histogram selection, streaming the row twice
      const int e = p->sparse_count <= kTopkThreads ? 1 : (p->sparse_count <= 2 * kTopkThreads ? 2 : 4);
      if (e == 1) li_topk_bins_stream_kernel<T, 1><<<(unsigned)rown, kTopkThreads, 0, st>>>(d, scores, ld);
      else if (e == 2) li_topk_bins_stream_kernel<T, 2><<<(unsigned)rown, kTopkThreads, 0, st>>>(d, scores, ld);
      else li_topk_bins_stream_kernel<T, 4><<<(unsigned)rown, kTopkThreads, 0, st>>>(d, scores, ld);
    } else {
      int32_t cap = 1;
      while (cap < p->sparse_count) cap <<= 1;
      const size_t smem = (size_t)cap * 8 + (size_t)kTopkKeyCache * 4;
      cudaError_t e;
      if (rank16) {
        e = cudaFuncSetAttribute(li_topk_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return DSA_ERR_CUDA;
        li_topk_kernel<T, true><<<(unsigned)rown, kTopkThreads, smem, st>>>(d, scores, ld, cap);
      } else {
        e = cudaFuncSetAttribute(li_topk_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return DSA_ERR_CUDA;
        li_topk_kernel<T, false><<<(unsigned)rown, kTopkThreads, smem, st>>>(d, scores, ld, cap);
      }
    }
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
    count_launch();
  }
  return DSA_OK;
}

static int sfa_validate(const DsaSfaParams* p) {
  if (p == nullptr) return DSA_ERR_NULL;
  if (p->struct_size != sizeof(DsaSfaParams)) return DSA_ERR_STRUCT;
  if (!p->query || !p->query_rope || !p->key || !p->key_rope || !p->sparse_indices || !p->out) return DSA_ERR_NULL;
  if (p->return_lse && (!p->softmax_max || !p->softmax_sum)) return DSA_ERR_NULL;
  if (p->layout_q != DSA_LAYOUT_BSND && p->layout_q != DSA_LAYOUT_TND) return DSA_ERR_VALUE;
  if (p->layout_kv < DSA_LAYOUT_BSND || p->layout_kv > DSA_LAYOUT_PA_BSND) return DSA_ERR_VALUE;
  if (p->dtype != DSA_DTYPE_BF16 && p->dtype != DSA_DTYPE_FP16) return DSA_ERR_VALUE;
  // shape guards of sparse_flash_attention_triton.py:1391-1398 (head count relaxed to any n1 >= 1)
  if (p->d != 128 && p->d != 256 && p->d != 512) return DSA_ERR_VALUE;
  if (p->d_rope != 64) return DSA_ERR_VALUE;
  if (p->batch < 1 || p->s1 < 0 || p->s2 < 0 || p->n1 < 1) return DSA_ERR_VALUE;
  if (p->sparse_mode != 0 && p->sparse_mode != 3) return DSA_ERR_VALUE;
  const int bs = p->sparse_block_size;
  if (bs < 1 || bs > 128 || (bs & (bs - 1)) != 0) return DSA_ERR_VALUE;  // :1349-1351
  if (p->sparse_count < 1) return DSA_ERR_VALUE;
  if (p->layout_q == DSA_LAYOUT_TND && (!p->seq_q || !p->seq_q_cumulative)) return DSA_ERR_VALUE;
  if (p->layout_kv == DSA_LAYOUT_TND && (!p->seq_k || !p->seq_k_cumulative)) return DSA_ERR_VALUE;
  if (p->layout_kv == DSA_LAYOUT_PA_BSND && (!p->block_table || p->block_size < 1 || p->max_blocks < 1 || !p->seq_k))
    return DSA_ERR_VALUE;
  if (p->kernel < DSA_KERNEL_AUTO || p->kernel > DSA_KERNEL_TENSOR) return DSA_ERR_VALUE;
  return DSA_OK;
}

static SfaDev sfa_dev(const DsaSfaParams* p) {
  SfaDev d;
  d.seq.seq_q = p->seq_q; d.seq.seq_k = p->seq_k; d.seq.block_table = p->block_table;
  d.seq.layout_q = p->layout_q; d.seq.layout_k = p->layout_kv;
  d.seq.seq_q_cum = p->seq_q_cumulative; d.seq.seq_k_cum = p->seq_k_cumulative;
  d.seq.batch = p->batch; d.seq.s1 = p->s1; d.seq.s2 = p->s2;
  d.seq.block_size = p->block_size; d.seq.max_blocks = p->max_blocks;
  d.seq.sparse_mode = p->sparse_mode;
  d.seq.key_rows = p->key_rows;
  d.query = p->query; d.query_rope = p->query_rope; d.key = p->key; d.key_rope = p->key_rope;
  d.sparse_indices = p->sparse_indices;
  d.out = p->out; d.softmax_max = p->softmax_max; d.softmax_sum = p->softmax_sum;
  d.rows = p->layout_q == DSA_LAYOUT_TND ? p->s1 : p->batch * p->s1;
  d.n1 = p->n1; d.d = p->d; d.d_rope = p->d_rope;
  d.sparse_count = p->sparse_count; d.sparse_block_size = p->sparse_block_size;
  d.return_lse = p->return_lse;
  d.scale = p->scale;
  return d;
}

template <typename T>
static int sfa_launch_simt(const DsaSfaParams* p, cudaStream_t st) {
  SfaDev d = sfa_dev(p);
  if (d.rows == 0) return DSA_OK;
  const size_t smem = (size_t)(kSfaSimtHeads + kSfaSimtKeys) * (p->d + p->d_rope + kSfaSimtPad) * sizeof(T);
  if (cudaFuncSetAttribute(sfa_fwd_mma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return DSA_ERR_CUDA;
  const unsigned gy = (unsigned)((p->n1 + kSfaSimtHeads - 1) / kSfaSimtHeads);
  dim3 grid((unsigned)d.rows, gy, 1);
  sfa_fwd_mma_kernel<T><<<grid, kSfaSimtThreads, smem, st>>>(d);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  count_launch();
  return DSA_OK;
}

// A wait that nothing satisfies, with a short limit: one thread waits on an mbarrier that no one
// ever arrives on (no copy or MMA is in flight), gives up and reports it the way the tensor-core
// kernels do (status word 1).  Used to test the failure path end to end without faulting a GPU.
__global__ void selftest_wait_timeout_kernel(int32_t* status, uint32_t polls) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    abort_flag = 0;
    ptx::mbar_fence_init();
    bool got = false;
    for (uint32_t i = 0; i < polls && !got; ++i) got = ptx::mbar_try_wait(&bar, 0);
    if (!got) atomicExch(status, 1);
  }
}

// ---------------------------------------------------------------------------------------------
// Attention backward: validation and launch
// ---------------------------------------------------------------------------------------------
static int sfa_grad_validate(const DsaSfaGradParams* p) {
  if (p == nullptr) return DSA_ERR_NULL;
  if (p->struct_size != sizeof(DsaSfaGradParams)) return DSA_ERR_STRUCT;
  if (!p->query || !p->query_rope || !p->key || !p->key_rope || !p->sparse_indices || !p->d_out || !p->out ||
      !p->softmax_max || !p->softmax_sum || !p->d_query || !p->d_query_rope || !p->d_key || !p->d_key_rope ||
      !p->d_value)
    return DSA_ERR_NULL;
  if (p->layout_q != DSA_LAYOUT_BSND && p->layout_q != DSA_LAYOUT_TND) return DSA_ERR_VALUE;
  if (p->layout_kv != DSA_LAYOUT_BSND && p->layout_kv != DSA_LAYOUT_TND) return DSA_ERR_VALUE;
  if (p->dtype != DSA_DTYPE_BF16 && p->dtype != DSA_DTYPE_FP16) return DSA_ERR_VALUE;
  // shape guards of sparse_flash_attention_grad_triton.py:587-594 (head count relaxed to any n1 >= 1)
  if (p->d != 128 && p->d != 256 && p->d != 512) return DSA_ERR_VALUE;
  if (p->d_rope != 64) return DSA_ERR_VALUE;
  if (p->batch < 1 || p->s1 < 0 || p->s2 < 0 || p->n1 < 1) return DSA_ERR_VALUE;
  if (p->sparse_mode != 0 && p->sparse_mode != 3) return DSA_ERR_VALUE;  // :552-553
  const int bs = p->sparse_block_size;
  if (bs < 1 || bs > 128 || (bs & (bs - 1)) != 0) return DSA_ERR_VALUE;  // :560-562
  if (p->sparse_count < 1 || p->key_rows < 0) return DSA_ERR_VALUE;
  if (p->layout_q == DSA_LAYOUT_TND && (!p->seq_q || !p->seq_q_cumulative)) return DSA_ERR_VALUE;
  if (p->layout_kv == DSA_LAYOUT_TND && (!p->seq_k || !p->seq_k_cumulative)) return DSA_ERR_VALUE;
  if (p->kernel != DSA_KERNEL_AUTO && p->kernel != DSA_KERNEL_PORTABLE && p->kernel != DSA_KERNEL_TENSOR)
    return DSA_ERR_UNSUPPORTED;
  return DSA_OK;
}

// 32 heads per block when there are more than 16 (half the scatter-adds per query row), else 16.
template <typename T, int D>
static int sfa_grad_mma_launch(const SfaGradDev& d, int n1, cudaStream_t st) {
  if (n1 > 16) {
    const size_t smem = sfa_grad_mma_smem_bytes<2, D>(sizeof(T));
    if (cudaFuncSetAttribute(sfa_bwd_mma_kernel<T, 2, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DSA_ERR_CUDA;
    dim3 grid((unsigned)d.rows, (unsigned)((n1 + 31) / 32), 1);
    sfa_bwd_mma_kernel<T, 2, D><<<grid, 512, smem, st>>>(d);
  } else {
    const size_t smem = sfa_grad_mma_smem_bytes<1, D>(sizeof(T));
    if (cudaFuncSetAttribute(sfa_bwd_mma_kernel<T, 1, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DSA_ERR_CUDA;
    dim3 grid((unsigned)d.rows, 1, 1);
    sfa_bwd_mma_kernel<T, 1, D><<<grid, 256, smem, st>>>(d);
  }
  return DSA_OK;
}

template <typename T>
static int sfa_grad_launch(const DsaSfaGradParams* p, float* acc, cudaStream_t st) {
  SfaGradDev d;
  d.seq.seq_q = p->seq_q; d.seq.seq_k = p->seq_k; d.seq.block_table = nullptr;
  d.seq.layout_q = p->layout_q; d.seq.layout_k = p->layout_kv;
  d.seq.seq_q_cum = p->seq_q_cumulative; d.seq.seq_k_cum = p->seq_k_cumulative;
  d.seq.batch = p->batch; d.seq.s1 = p->s1; d.seq.s2 = p->s2;
  d.seq.block_size = 0; d.seq.max_blocks = 0;
  d.seq.sparse_mode = p->sparse_mode;
  d.seq.key_rows = p->key_rows;
  d.query = p->query; d.query_rope = p->query_rope; d.key = p->key; d.key_rope = p->key_rope;
  d.sparse_indices = p->sparse_indices;
  d.d_out = p->d_out; d.out = p->out; d.softmax_max = p->softmax_max; d.softmax_sum = p->softmax_sum;
  d.d_query = p->d_query; d.d_query_rope = p->d_query_rope;
  d.dk_acc = acc;
  d.dv_acc = acc + p->key_rows * (p->d + p->d_rope);
  d.rows = p->layout_q == DSA_LAYOUT_TND ? p->s1 : p->batch * p->s1;
  d.n1 = p->n1; d.d = p->d; d.d_rope = p->d_rope;
  d.sparse_count = p->sparse_count; d.sparse_block_size = p->sparse_block_size;
  d.scale = p->scale;
  if (d.rows > 0) {
    const unsigned gy = (unsigned)((p->n1 + kSfaGradHeads - 1) / kSfaGradHeads);
    dim3 grid((unsigned)d.rows, gy, 1);
    // the contractions run on the tensor cores (mma.sync); on request the CUDA-core kernel
    if (p->kernel != DSA_KERNEL_PORTABLE) {
      int rc;
      if (p->d == 512) rc = sfa_grad_mma_launch<T, 512>(d, p->n1, st);
      else if (p->d == 256) rc = sfa_grad_mma_launch<T, 256>(d, p->n1, st);
      else rc = sfa_grad_mma_launch<T, 128>(d, p->n1, st);
      if (rc != DSA_OK) return rc;
    } else {
      const size_t smem = sfa_grad_smem_bytes(p->d, p->d_rope, sizeof(T));
      if (cudaFuncSetAttribute(sfa_bwd_simt_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
          cudaSuccess)
        return DSA_ERR_CUDA;
      sfa_bwd_simt_kernel<T><<<grid, kSfaGradThreads, smem, st>>>(d);
    }
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
    count_launch();
  }
  if (p->key_rows > 0) {
    const int64_t total = p->key_rows * (int64_t)(2 * p->d + p->d_rope);
    const unsigned blocks = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 16);
    sfa_bwd_finalize_kernel<T><<<blocks, 256, 0, st>>>(d.dk_acc, d.dv_acc, (T*)p->d_key, (T*)p->d_key_rope,
                                                      (T*)p->d_value, p->key_rows, p->d, p->d_rope);
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
    count_launch();
  }
  return DSA_OK;
}


// ---------------------------------------------------------------------------------------------
// Indexer KL-loss backward: validation and launch
// ---------------------------------------------------------------------------------------------
// Slots per query row: topk for the sparse operator, every key for the dense one.
static int64_t sli_slots(const DsaSliGradParams* p) { return p->dense ? p->s2 : p->topk; }

static int sli_grad_validate(const DsaSliGradParams* p) {
  if (p == nullptr) return DSA_ERR_NULL;
  if (p->struct_size != sizeof(DsaSliGradParams)) return DSA_ERR_STRUCT;
  if (!p->query || !p->key || !p->query_index || !p->key_index || !p->weights ||
      (!p->dense && !p->sparse_indices) || !p->softmax_max || !p->softmax_sum || !p->d_query_index || !p->d_key_index || !p->d_weights || !p->loss)
    return DSA_ERR_NULL;
  if (p->d_rope != 0 && (!p->query_rope || !p->key_rope)) return DSA_ERR_NULL;
  if (p->dtype != DSA_DTYPE_BF16 && p->dtype != DSA_DTYPE_FP16) return DSA_ERR_VALUE;
  if (p->dtype_w < DSA_DTYPE_BF16 || p->dtype_w > DSA_DTYPE_FP32) return DSA_ERR_VALUE;
  // shapes the reference is specified for (test_sli_grad_kl_loss_triton.py:43-45), any head counts
  if (p->d != 128 && p->d != 256 && p->d != 512) return DSA_ERR_VALUE;
  if (p->d_idx != 128 && p->d_idx != 256 && p->d_idx != 512) return DSA_ERR_VALUE;
  if (p->d_rope != 0 && p->d_rope != 64) return DSA_ERR_VALUE;
  if (p->batch < 1 || p->s1 < 0 || p->s2 < 1 || p->n1 < 1 || p->g < 1) return DSA_ERR_VALUE;
  if (p->dense) {
    if (p->n2 < 1 || p->n1 % p->n2 != 0) return DSA_ERR_VALUE;
    if ((p->softmax_max_index == nullptr) != (p->softmax_sum_index == nullptr)) return DSA_ERR_NULL;
  } else {
    if (p->n2 != 1 && p->n2 != 0) return DSA_ERR_VALUE;
    if (p->topk < 1) return DSA_ERR_VALUE;
  }
  if (p->kernel != DSA_KERNEL_AUTO && p->kernel != DSA_KERNEL_PORTABLE) return DSA_ERR_UNSUPPORTED;
  return DSA_OK;
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

template <typename T>
static int sli_grad_launch(const DsaSliGradParams* p, char* ws, int32_t* status, cudaStream_t st) {
  SliGradDev d;
  const int64_t rows = (int64_t)p->batch * p->s1;
  const int64_t key_elems = (int64_t)p->batch * p->s2 * p->d_idx;
  d.query = p->query; d.query_rope = p->d_rope ? p->query_rope : nullptr;
  d.key = p->key; d.key_rope = p->d_rope ? p->key_rope : nullptr;
  d.query_index = p->query_index; d.key_index = p->key_index; d.weights = p->weights;
  d.sparse_indices = p->dense ? nullptr : p->sparse_indices;
  d.softmax_max = p->softmax_max; d.softmax_sum = p->softmax_sum;
  d.act_q = p->seq_q; d.act_k = p->seq_k;
  const int32_t slots = (int32_t)sli_slots(p);
  d.d_query_index = p->d_query_index; d.d_weights = p->d_weights; d.d_key_index = p->d_key_index; d.loss = p->loss;
  const size_t buf_bytes = align256((size_t)rows * slots * 4);
  d.di = reinterpret_cast<float*>(ws);
  d.p_buf = reinterpret_cast<float*>(ws + buf_bytes);
  d.loss_parts = reinterpret_cast<float*>(ws + 2 * buf_bytes);
  float* stats = reinterpret_cast<float*>((char*)d.loss_parts + align256((size_t)rows * 4));
  d.dki_acc = reinterpret_cast<float*>((char*)stats + align256((size_t)rows * 8));
  d.stats_given = (p->dense && p->softmax_max_index) ? 1 : 0;
  d.index_max = d.stats_given ? const_cast<float*>(p->softmax_max_index) : stats;
  d.index_sum = d.stats_given ? const_cast<float*>(p->softmax_sum_index) : stats + rows;
  d.lse_only = 0;
  d.batch = p->batch; d.s1 = p->s1; d.s2 = p->s2; d.n1 = p->n1; d.n2 = p->dense ? p->n2 : 1;
  d.d = p->d; d.d_rope = p->d_rope;
  d.g = p->g; d.d_idx = p->d_idx; d.topk = slots; d.dtype_w = p->dtype_w;
  d.scale = p->scale;
  if (cudaMemsetAsync(d.dki_acc, 0, (size_t)key_elems * 4, st) != cudaSuccess) return DSA_ERR_CUDA;
  if (rows > 0 && cudaMemsetAsync(d.di, 0, 2 * buf_bytes, st) != cudaSuccess) return DSA_ERR_CUDA;
  if (rows > 0) {
    const int stride = std::max(p->d + p->d_rope, p->d_idx) + kSliPad;
    // teacher blocks of 32 heads when a side has more than 16 (half the key gathers per row)
    const int hb = (d.n1 / d.n2 > kSliHeads || d.g > kSliHeads) ? 2 * kSliHeads : kSliHeads;
    const size_t smem_a = (size_t)(hb + kSliTeacherKeys) * stride * sizeof(T);
    const size_t smem_d = (size_t)(kSliHeads + kSliTeacherKeys) * stride * sizeof(T);
    // gradient blocks of 32 heads for d_idx = 128 (both head tiles' dQI accumulators fit in registers)
    const int hg = (d.g > kSliHeads && p->d_idx == 128) ? 2 * kSliHeads : kSliHeads;
    const size_t smem_b = (size_t)(hg + kSliTeacherKeys) * (p->d_idx + kSliPad) * sizeof(T);
    if (cudaFuncSetAttribute(sli_teacher_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a) !=
            cudaSuccess ||
        cudaFuncSetAttribute(sli_teacher_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a) !=
            cudaSuccess ||
        cudaFuncSetAttribute(sli_grad_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b) !=
            cudaSuccess ||
        cudaFuncSetAttribute(sli_grad_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b) !=
            cudaSuccess)
      return DSA_ERR_CUDA;
    // Dense operator: the index scores of all visible keys are the lightning indexer's scores; when
    // the shape is one the tcgen05 scoring kernel takes, it writes them (row stride = s2) and the
    // CUDA-core pass below only does the attention side.
    bool index_done = false;
    if (p->dense && p->s2 % 4 == 0 && status != nullptr) {
      DsaLiParams l = {};
      l.struct_size = sizeof(DsaLiParams);
      l.kernel = DSA_KERNEL_AUTO;
      l.query = p->query_index; l.key = p->key_index; l.weights = p->weights;
      l.seq_q = p->seq_q; l.seq_k = p->seq_k;
      l.out_indices = (int32_t*)d.loss_parts;   // (not written: the top-k phase does not run)
      l.layout_q = DSA_LAYOUT_BSND; l.layout_k = DSA_LAYOUT_BSND;
      l.dtype_qk = p->dtype; l.dtype_w = p->dtype_w;
      l.batch = p->batch; l.s1 = p->s1; l.s2 = p->s2; l.n1 = p->g; l.n2 = 1; l.d = p->d_idx;
      l.sparse_count = 1; l.sparse_mode = 3; l.rank_mode = DSA_RANK_IO_DTYPE; l.phases = DSA_PHASE_SCORE;
      l.key_rows = (int64_t)p->batch * p->s2;
      if (li_validate(&l) == DSA_OK && li_takes_tensor_path(&l)) {
        int rc = li_launch<T>(&l, d.di, st, status);
        if (rc != DSA_OK) return rc;
        index_done = true;
      }
    }
    // Dense operator with fewer than 16 query heads per key head: blocks of 16 (row, head) pairs
    // share the keys they walk over; the per-row kernel then only does the index side, if any.
    const int grp = d.n1 / d.n2;
    const bool pair_blocks = p->dense && grp < kSliHeads && kSliHeads % grp == 0;
    if (pair_blocks) {
      if (cudaFuncSetAttribute(sli_dense_teacher_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem_d) != cudaSuccess)
        return DSA_ERR_CUDA;
      const int rpb = kSliHeads / grp;
      dim3 grid_d((unsigned)(p->batch * ((p->s1 + rpb - 1) / rpb)), (unsigned)d.n2, 1);
      sli_dense_teacher_kernel<T><<<grid_d, kSliThreads, smem_d, st>>>(d, stride);
      if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
      count_launch();
    }
    SliGradDev dt = d;
    if (pair_blocks) dt.lse_only = 1;   // index chunks only
    const unsigned chunks_t =
        (unsigned)((pair_blocks ? 0 : sli_att_chunks(d.n1, d.n2, hb)) + (index_done ? 0 : sli_idx_chunks(d.g, hb)));
    if (chunks_t > 0) {
      dim3 grid_t((unsigned)rows, chunks_t, 1);
      if (hb > kSliHeads) sli_teacher_kernel<T, 2><<<grid_t, kSliThreads, smem_a, st>>>(dt, stride);
      else sli_teacher_kernel<T, 1><<<grid_t, kSliThreads, smem_a, st>>>(dt, stride);
      if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
      count_launch();
    }
    sli_student_kernel<<<(unsigned)rows, kSliThreads, 0, st>>>(d);
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
    dim3 grid((unsigned)rows, (unsigned)sli_idx_chunks(d.g, hg), 1);
    if (hg > kSliHeads) sli_grad_kernel<T, 2><<<grid, kSliThreads, smem_b, st>>>(d);
    else sli_grad_kernel<T, 1><<<grid, kSliThreads, smem_b, st>>>(d);
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
    count_launch(2);
  }
  const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>((key_elems + 255) / 256, 148 * 16));
  sli_finalize_kernel<T><<<blocks, 256, 0, st>>>(d, key_elems, (int32_t)rows);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  count_launch();
  return DSA_OK;
}
// The dense index scores are the lightning indexer's scores: the same problem as an indexer call
// (BSND, rightDownCausal, per-batch lengths) stopped after the scoring phase.
static DsaLiParams dense_lse_as_li(const DsaDenseLseParams* p) {
  DsaLiParams l = {};
  l.struct_size = sizeof(DsaLiParams);
  l.kernel = DSA_KERNEL_AUTO;
  l.query = p->query_index; l.key = p->key_index; l.weights = p->weights;
  l.seq_q = p->seq_q; l.seq_k = p->seq_k;
  l.out_indices = (int32_t*)p->softmax_max_index;   // (not written: the top-k phase does not run)
  l.layout_q = DSA_LAYOUT_BSND; l.layout_k = DSA_LAYOUT_BSND;
  l.dtype_qk = p->dtype; l.dtype_w = p->dtype_w;
  l.batch = p->batch; l.s1 = p->s1; l.s2 = p->s2; l.n1 = p->g; l.n2 = 1; l.d = p->d_idx;
  l.sparse_count = 1; l.sparse_mode = 3; l.rank_mode = DSA_RANK_IO_DTYPE; l.phases = DSA_PHASE_SCORE;
  l.key_rows = (int64_t)p->batch * p->s2;
  return l;
}

template <typename T>
static int dense_lse_launch(const DsaDenseLseParams* p, float* scratch, int32_t* status, cudaStream_t st) {
  SliGradDev d = {};
  d.query_index = p->query_index; d.key_index = p->key_index; d.weights = p->weights;
  d.act_q = p->seq_q; d.act_k = p->seq_k;
  d.index_max = p->softmax_max_index; d.index_sum = p->softmax_sum_index;
  d.batch = p->batch; d.s1 = p->s1; d.s2 = p->s2; d.n1 = 1; d.n2 = 1; d.g = p->g; d.d_idx = p->d_idx;
  d.topk = p->s2; d.dtype_w = p->dtype_w; d.lse_only = 1;
  const int64_t rows = (int64_t)p->batch * p->s1;
  if (rows == 0) return DSA_OK;
  const DsaLiParams lp = dense_lse_as_li(p);
  if (li_validate(&lp) == DSA_OK && li_takes_tensor_path(&lp)) {
    // tcgen05 scoring kernel, then one reduction per row
    int rc = li_launch<T>(&lp, scratch, st, status);
    if (rc != DSA_OK) return rc;
    sli_lse_rows_kernel<<<(unsigned)rows, kSliThreads, 0, st>>>(d, scratch, li_score_ld(&lp));
    if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
    count_launch();
    return DSA_OK;
  }
  d.di = scratch;
  if (cudaMemsetAsync(scratch, 0, (size_t)rows * p->s2 * 4, st) != cudaSuccess) return DSA_ERR_CUDA;
  const int stride = p->d_idx + kSliPad;
  const int hb = p->g > kSliHeads ? 2 * kSliHeads : kSliHeads;
  const size_t smem = (size_t)(hb + kSliTeacherKeys) * stride * sizeof(T);
  if (cudaFuncSetAttribute(sli_teacher_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
          cudaSuccess ||
      cudaFuncSetAttribute(sli_teacher_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
          cudaSuccess)
    return DSA_ERR_CUDA;
  dim3 grid((unsigned)rows, (unsigned)sli_idx_chunks(p->g, hb), 1);
  if (hb > kSliHeads) sli_teacher_kernel<T, 2><<<grid, kSliThreads, smem, st>>>(d, stride);
  else sli_teacher_kernel<T, 1><<<grid, kSliThreads, smem, st>>>(d, stride);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  sli_student_kernel<<<(unsigned)rows, kSliThreads, 0, st>>>(d);
  if (cudaGetLastError() != cudaSuccess) return DSA_ERR_CUDA;
  count_launch(2);
  return DSA_OK;
}

}  // namespace dsa

using namespace dsa;

extern "C" {

int dsa_abi_version(void) { return 7; }

unsigned long long dsa_kernel_launch_count(void) { return launch_counter().load(std::memory_order_relaxed); }

const char* dsa_status_string(int status) {
  switch (status) {
    case DSA_OK: return "ok";
    case DSA_ERR_NULL: return "a required pointer is NULL";
    case DSA_ERR_STRUCT: return "struct_size does not match the library (ABI mismatch)";
    case DSA_ERR_VALUE: return "argument outside the supported set";
    case DSA_ERR_WORKSPACE: return "workspace too small or not 256-byte aligned";
    case DSA_ERR_UNSUPPORTED: return "requested kernel variant cannot run this shape";
    case DSA_ERR_CUDA: return "a CUDA runtime call failed";
    case DSA_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
    case DSA_ERR_TOO_LARGE: return "size beyond a fixed maximum of the library";
    default: return "unknown status";
  }
}

int dsa_li_uses_tensor_path(const DsaLiParams* p) {
  if (li_validate(p) != DSA_OK) return 0;
  return li_takes_tensor_path(p) ? 1 : 0;
}

int dsa_sfa_uses_tensor_path(const DsaSfaParams* p) {
  if (sfa_validate(p) != DSA_OK) return 0;
  return (p->kernel != DSA_KERNEL_PORTABLE && sfa_sm100_eligible(p)) ? 1 : 0;
}

int dsa_li_workspace_bytes(const DsaLiParams* p, size_t* out_bytes) {
  int st = li_validate(p);
  if (st != DSA_OK) return st;
  if (!out_bytes) return DSA_ERR_NULL;
  const int64_t rown = li_rows(p) * p->n2;
  *out_bytes = kWorkspaceHeader + (size_t)round_up(rown * li_score_ld(p) * 4, 256);
  return DSA_OK;
}

int dsa_li_forward(const DsaLiParams* p, void* workspace, size_t workspace_bytes, void* stream) {
  int st = li_validate(p);
  if (st != DSA_OK) return st;
  size_t need = 0;
  dsa_li_workspace_bytes(p, &need);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255u) != 0) return DSA_ERR_WORKSPACE;
  if (p->kernel == DSA_KERNEL_TENSOR && !dsa_li_uses_tensor_path(p)) return DSA_ERR_UNSUPPORTED;
  cudaStream_t cs = (cudaStream_t)stream;
  if (cudaMemsetAsync(workspace, 0, kWorkspaceHeader, cs) != cudaSuccess) return DSA_ERR_CUDA;
  float* scores = reinterpret_cast<float*>((char*)workspace + kWorkspaceHeader);
  if (p->dtype_qk == DSA_DTYPE_BF16) return li_launch<__nv_bfloat16>(p, scores, cs, (int32_t*)workspace);
  return li_launch<__half>(p, scores, cs, (int32_t*)workspace);
}

int dsa_sfa_workspace_bytes(const DsaSfaParams* p, size_t* out_bytes) {
  int st = sfa_validate(p);
  if (st != DSA_OK) return st;
  if (!out_bytes) return DSA_ERR_NULL;
  *out_bytes = kWorkspaceHeader + (dsa_sfa_uses_tensor_path(p) ? sfa_sm100_workspace_bytes(p) : 0);
  return DSA_OK;
}

int dsa_sfa_forward(const DsaSfaParams* p, void* workspace, size_t workspace_bytes, void* stream) {
  int st = sfa_validate(p);
  if (st != DSA_OK) return st;
  size_t need = 0;
  dsa_sfa_workspace_bytes(p, &need);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255u) != 0) return DSA_ERR_WORKSPACE;
  if (p->kernel == DSA_KERNEL_TENSOR && !dsa_sfa_uses_tensor_path(p)) return DSA_ERR_UNSUPPORTED;
  cudaStream_t cs = (cudaStream_t)stream;
  if (dsa_sfa_uses_tensor_path(p)) {
    SfaDev d = sfa_dev(p);
    if (d.rows > 0)   // (the pre-pass kernel clears the header)
      return sfa_sm100_launch(p, d, (int32_t*)workspace, (char*)workspace + kWorkspaceHeader, cs);
  }
  if (cudaMemsetAsync(workspace, 0, kWorkspaceHeader, cs) != cudaSuccess) return DSA_ERR_CUDA;
  if (dsa_sfa_uses_tensor_path(p)) return DSA_OK;   // no rows
  if (p->dtype == DSA_DTYPE_BF16) return sfa_launch_simt<__nv_bfloat16>(p, cs);
  return sfa_launch_simt<__half>(p, cs);
}

// ---------------------------------------------------------------------------------------------
// Attention backward
// ---------------------------------------------------------------------------------------------
int dsa_sfa_grad_workspace_bytes(const DsaSfaGradParams* p, size_t* out_bytes) {
  int st = sfa_grad_validate(p);
  if (st != DSA_OK) return st;
  if (!out_bytes) return DSA_ERR_NULL;
  *out_bytes = kWorkspaceHeader + (size_t)p->key_rows * (size_t)(2 * p->d + p->d_rope) * sizeof(float);
  return DSA_OK;
}

int dsa_sfa_grad(const DsaSfaGradParams* p, void* workspace, size_t workspace_bytes, void* stream) {
  int st = sfa_grad_validate(p);
  if (st != DSA_OK) return st;
  size_t need = 0;
  dsa_sfa_grad_workspace_bytes(p, &need);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255u) != 0) return DSA_ERR_WORKSPACE;
  cudaStream_t cs = (cudaStream_t)stream;
  if (cudaMemsetAsync(workspace, 0, need, cs) != cudaSuccess) return DSA_ERR_CUDA;
  float* acc = reinterpret_cast<float*>((char*)workspace + kWorkspaceHeader);
  if (p->dtype == DSA_DTYPE_BF16) return sfa_grad_launch<__nv_bfloat16>(p, acc, cs);
  return sfa_grad_launch<__half>(p, acc, cs);
}

static int dense_lse_validate(const DsaDenseLseParams* p) {
  if (p == nullptr) return DSA_ERR_NULL;
  if (p->struct_size != sizeof(DsaDenseLseParams)) return DSA_ERR_STRUCT;
  if (!p->query_index || !p->key_index || !p->weights || !p->softmax_max_index || !p->softmax_sum_index)
    return DSA_ERR_NULL;
  if (p->dtype != DSA_DTYPE_BF16 && p->dtype != DSA_DTYPE_FP16) return DSA_ERR_VALUE;
  if (p->dtype_w < DSA_DTYPE_BF16 || p->dtype_w > DSA_DTYPE_FP32) return DSA_ERR_VALUE;
  if (p->d_idx != 128 && p->d_idx != 256 && p->d_idx != 512) return DSA_ERR_VALUE;
  if (p->batch < 1 || p->s1 < 0 || p->s2 < 1 || p->g < 1) return DSA_ERR_VALUE;
  if ((int64_t)p->batch * p->s1 > 0x7FFFFFFF) return DSA_ERR_TOO_LARGE;
  return DSA_OK;
}

int dsa_dense_li_lse_workspace_bytes(const DsaDenseLseParams* p, size_t* out_bytes) {
  int st = dense_lse_validate(p);
  if (st != DSA_OK) return st;
  if (!out_bytes) return DSA_ERR_NULL;
  const DsaLiParams lp = dense_lse_as_li(p);
  size_t scores = (size_t)p->batch * p->s1 * p->s2 * 4;
  if (li_validate(&lp) == DSA_OK)
    scores = std::max(scores, (size_t)round_up(li_rows(&lp) * li_score_ld(&lp) * 4, 256));
  *out_bytes = kWorkspaceHeader + scores;
  return DSA_OK;
}

int dsa_dense_li_lse(const DsaDenseLseParams* p, void* workspace, size_t workspace_bytes, void* stream) {
  int st = dense_lse_validate(p);
  if (st != DSA_OK) return st;
  size_t need = 0;
  dsa_dense_li_lse_workspace_bytes(p, &need);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255u) != 0) return DSA_ERR_WORKSPACE;
  cudaStream_t cs = (cudaStream_t)stream;
  if (cudaMemsetAsync(workspace, 0, kWorkspaceHeader, cs) != cudaSuccess) return DSA_ERR_CUDA;
  float* scratch = reinterpret_cast<float*>((char*)workspace + kWorkspaceHeader);
  if (p->dtype == DSA_DTYPE_BF16) return dense_lse_launch<__nv_bfloat16>(p, scratch, (int32_t*)workspace, cs);
  return dense_lse_launch<__half>(p, scratch, (int32_t*)workspace, cs);
}

int dsa_sli_grad_workspace_bytes(const DsaSliGradParams* p, size_t* out_bytes) {
  int st = sli_grad_validate(p);
  if (st != DSA_OK) return st;
  if (!out_bytes) return DSA_ERR_NULL;
  const size_t rows = (size_t)p->batch * p->s1;
  *out_bytes = kWorkspaceHeader + 2 * align256(rows * (size_t)sli_slots(p) * 4) + align256(rows * 4) +
               align256(rows * 8) + (size_t)p->batch * p->s2 * p->d_idx * 4;
  return DSA_OK;
}

int dsa_sli_grad(const DsaSliGradParams* p, void* workspace, size_t workspace_bytes, void* stream) {
  int st = sli_grad_validate(p);
  if (st != DSA_OK) return st;
  size_t need = 0;
  dsa_sli_grad_workspace_bytes(p, &need);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255u) != 0) return DSA_ERR_WORKSPACE;
  if ((int64_t)p->batch * p->s1 > 0x7FFFFFFF) return DSA_ERR_TOO_LARGE;
  cudaStream_t cs = (cudaStream_t)stream;
  if (cudaMemsetAsync(workspace, 0, kWorkspaceHeader, cs) != cudaSuccess) return DSA_ERR_CUDA;
  char* ws = (char*)workspace + kWorkspaceHeader;
  if (p->dtype == DSA_DTYPE_BF16) return sli_grad_launch<__nv_bfloat16>(p, ws, (int32_t*)workspace, cs);
  return sli_grad_launch<__half>(p, ws, (int32_t*)workspace, cs);
}

// ---------------------------------------------------------------------------------------------
// Indexer entry point for callers that cannot hand over a workspace and must not allocate.
// The fp32 score rows live in a fixed array inside the library image instead.
// ---------------------------------------------------------------------------------------------
#define DSA_LI_STATIC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_li_static_scratch[kWorkspaceHeader + DSA_LI_STATIC_SCRATCH_BYTES];

// Device address of the array, resolved once per device.  In host code the array's name is only
// a handle for the runtime, never a pointer a kernel may use.
static void* g_li_static_ptr[64] = {nullptr};

static int li_static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DSA_ERR_CUDA;
  void* ptr = __atomic_load_n(&g_li_static_ptr[dev], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {
    if (cudaGetSymbolAddress(&ptr, g_li_static_scratch) != cudaSuccess || ptr == nullptr) return DSA_ERR_CUDA;
    __atomic_store_n(&g_li_static_ptr[dev], ptr, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return DSA_OK;
}

size_t dsa_li_static_scratch_bytes(void) { return (size_t)DSA_LI_STATIC_SCRATCH_BYTES; }

int dsa_li_forward_static(const DsaLiParams* p, void* stream) {
  int st = li_validate(p);
  if (st != DSA_OK) return st;
  const int64_t score_bytes = li_rows(p) * p->n2 * li_score_ld(p) * 4;
  if (score_bytes > (int64_t)DSA_LI_STATIC_SCRATCH_BYTES) return DSA_ERR_TOO_LARGE;
  if (p->kernel == DSA_KERNEL_TENSOR) return DSA_ERR_UNSUPPORTED;
  void* scratch = nullptr;
  st = li_static_scratch(&scratch);
  if (st != DSA_OK) return st;
  cudaStream_t cs = (cudaStream_t)stream;
  // the array keeps the previous call's bytes: the status word has to start at zero
  if (cudaMemsetAsync(scratch, 0, kWorkspaceHeader, cs) != cudaSuccess) return DSA_ERR_CUDA;
  float* scores = reinterpret_cast<float*>((char*)scratch + kWorkspaceHeader);
  if (p->dtype_qk == DSA_DTYPE_BF16) return li_launch<__nv_bfloat16>(p, scores, cs);
  return li_launch<__half>(p, scores, cs);
}

#ifdef DSA_TOPK_PROFILE
// Development aid (see li_topk.cuh): cycles per phase of one top-k CTA.
int dsa_debug_topk_profile(long long* out) {
  return cudaMemcpyFromSymbol(out, g_topk_prof, sizeof(long long) * 16) == cudaSuccess ? DSA_OK : DSA_ERR_CUDA;
}
#endif
#ifdef DSA_SFA_PROFILE
// development builds only: the attention kernel's cycle counters (128 values)
int dsa_debug_sfa_profile(long long* out) {
  return cudaMemcpyFromSymbol(out, g_sfa_prof, sizeof(long long) * 128) == cudaSuccess ? DSA_OK : DSA_ERR_CUDA;
}
#endif

int dsa_selftest_wait_timeout(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < kWorkspaceHeader || ((uintptr_t)workspace & 255u) != 0) return DSA_ERR_WORKSPACE;
  cudaStream_t cs = (cudaStream_t)stream;
  if (cudaMemsetAsync(workspace, 0, kWorkspaceHeader, cs) != cudaSuccess) return DSA_ERR_CUDA;
  selftest_wait_timeout_kernel<<<1, 32, 0, cs>>>((int32_t*)workspace, 64u);   // 64 polls of up to 8 us
  return cudaGetLastError() == cudaSuccess ? DSA_OK : DSA_ERR_CUDA;
}

int dsa_read_device_status(const void* workspace, void* stream) {
  if (!workspace) return DSA_ERR_NULL;
  int32_t word = 0;
  cudaStream_t cs = (cudaStream_t)stream;
  if (cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, cs) != cudaSuccess) return DSA_ERR_CUDA;
  if (cudaStreamSynchronize(cs) != cudaSuccess) return DSA_ERR_CUDA;
  return word == 0 ? DSA_OK : DSA_ERR_DEVICE_WAIT;
}

}  // extern "C"
