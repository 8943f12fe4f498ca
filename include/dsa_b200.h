/*
 * dsa_b200.h - C ABI of the B200 (sm_100a) DeepSeek-Sparse-Attention forward kernels.
 *
 * The library replaces the device side of two operators of WhFanatic/dsa_triton_ascend:
 *   lightning_indexer       (score kernel + top-k)   lightning_indexer_triton.py:466-554
 *   sparse_flash_attention  (forward)                sparse_flash_attention_triton.py:1295-1455
 * The reference reaches its kernels through `ms.ops._ms_pyfunc` cores that take typed
 * tensors plus scalars, write into caller-allocated buffers and report nothing from the
 * device (lightning_indexer_triton.py:386-417, sparse_flash_attention_triton.py:1160-1289).
 * This ABI keeps that contract: plain pointers and sizes, the caller owns every buffer
 * (inputs, outputs, workspace), calls are enqueued on the given CUDA stream and return
 * without synchronising.  All functions return 0 on success and a negative DSA_ERR_*
 * code otherwise; none throws, exits or allocates device memory (except the entry point
 * explicitly documented to own static device scratch).
 */
#ifndef DSA_B200_H_
#define DSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define DSA_OK 0
#define DSA_ERR_NULL (-1)         /* a required pointer is NULL                      */
#define DSA_ERR_STRUCT (-2)       /* struct_size does not match this library          */
#define DSA_ERR_VALUE (-3)        /* argument outside the supported set (ValueError)  */
#define DSA_ERR_WORKSPACE (-4)    /* workspace too small or misaligned                */
#define DSA_ERR_UNSUPPORTED (-5)  /* requested kernel variant cannot run this shape   */
#define DSA_ERR_CUDA (-6)         /* a CUDA runtime call failed (launch, attribute)   */
#define DSA_ERR_DEVICE_WAIT (-7)  /* a bounded device-side wait ran out (status word) */
#define DSA_ERR_TOO_LARGE (-8)    /* size beyond a documented fixed maximum           */

/* enums (plain ints in the structs) */
#define DSA_LAYOUT_BSND 0
#define DSA_LAYOUT_TND 1
#define DSA_LAYOUT_PA_BSND 2

#define DSA_DTYPE_BF16 0
#define DSA_DTYPE_FP16 1
#define DSA_DTYPE_FP32 2

#define DSA_RANK_IO_DTYPE 0 /* rank scores rounded to the q/k dtype (numpy golden)       */
#define DSA_RANK_FP32 1     /* rank raw fp32 scores (what the reference device path does) */

#define DSA_KERNEL_AUTO 0     /* tensor-core path when the shape is eligible, else portable */
#define DSA_KERNEL_PORTABLE 1 /* any-shape kernels (mma.sync / CUDA cores)                    */
#define DSA_KERNEL_TENSOR 2   /* tensor-core path (tcgen05 forward, mma.sync backward);
                                 DSA_ERR_UNSUPPORTED when the shape is not eligible         */

#define DSA_PHASE_SCORE 1
#define DSA_PHASE_TOPK 2
#define DSA_PHASE_ALL 3

/*
 * lightning_indexer.  Replaces _lightning_indexer_score_core + _stable_topk
 * (lightning_indexer_triton.py:386-417, 343-361) and the TND copy loops (:294-340).
 *
 *   score[row, n2, s2] = sum_{g in group n2} relu(Q[row, g, :] . K[s2, n2, :]) * W[row, g]
 * masked to the row's visible prefix, then the `sparse_count` best keys are emitted in
 * (score descending, position ascending) order; unused slots hold index -1 / value 0.
 *
 * Row numbering: BSND row = b * s1 + position, TND row = token.  Positions written to
 * out_indices are local to the row's own sequence (batch-local), as in the reference.
 */
typedef struct DsaLiParams {
  uint32_t struct_size; /* sizeof(DsaLiParams) */
  int32_t kernel;       /* DSA_KERNEL_*  */
  const void* query;    /* BSND [batch, s1, n1, d] | TND [s1(=T1), n1, d]                    */
  const void* key;      /* BSND [batch, s2, n2, d] | TND [T2, n2, d] | PA [blocks, block_size, n2, d] */
  const void* weights;  /* [rows, n1], dtype_w                                                */
  const int32_t* seq_q; /* [batch] lengths, or cumulative ends when seq_q_cumulative; NULL = s1 */
  const int32_t* seq_k; /* [batch] lengths, or cumulative ends when seq_k_cumulative; NULL = s2 */
  const int32_t* block_table; /* PA only: [batch, max_blocks], -1 = no block                  */
  int32_t* out_indices; /* [rows, n2, sparse_count]                                           */
  void* out_values;     /* [rows, n2, sparse_count] in dtype_qk; may be NULL if !return_value */
  int32_t layout_q;     /* DSA_LAYOUT_BSND | DSA_LAYOUT_TND                                    */
  int32_t layout_k;     /* DSA_LAYOUT_*                                                        */
  int32_t dtype_qk;     /* DSA_DTYPE_BF16 | DSA_DTYPE_FP16                                     */
  int32_t dtype_w;      /* DSA_DTYPE_BF16 | FP16 | FP32                                        */
  int32_t seq_q_cumulative;
  int32_t seq_k_cumulative;
  int32_t batch;
  int32_t s1;           /* BSND: S1; TND: total query tokens T1                                */
  int32_t s2;           /* BSND: S2; TND/PA: upper bound of any sequence's key length          */
  int32_t n1, n2, d;
  int32_t block_size, max_blocks; /* PA only */
  int32_t sparse_count;
  int32_t sparse_mode;  /* 0 full, 3 rightDownCausal */
  int32_t rank_mode;    /* DSA_RANK_* */
  int32_t return_value;
  int32_t phases;       /* DSA_PHASE_*; score-only and top-k-only share the workspace scores  */
  int64_t key_rows;     /* rows of the key tensor: batch*s2 (BSND), T2 (TND), blocks*block_size (PA) */
} DsaLiParams;

/*
 * sparse_flash_attention forward, MLA-absorb (value = key[..., :d]), one KV head.
 * Replaces _sfa_core and its three kernels (sparse_flash_attention_triton.py:1160-1289,
 * 324-962), the layout copy loops (:975-1033) and _expand_block_indices (:1036-1051).
 *
 * A slot j of a row selects token  idx[j / sparse_block_size] * sparse_block_size +
 * j % sparse_block_size; it takes part when idx != -1, token < threshold and token <
 * act_k, with threshold = act_k (mode 0) or act_k - act_q + position + 1 (mode 3)
 * (sparse_flash_attention_triton.py:392-398,465).  Rows without any valid slot produce
 * zeros in all three outputs.
 */
typedef struct DsaSfaParams {
  uint32_t struct_size; /* sizeof(DsaSfaParams) */
  int32_t kernel;       /* DSA_KERNEL_* */
  const void* query;      /* [rows, n1, d]        */
  const void* query_rope; /* [rows, n1, d_rope]   */
  const void* key;        /* BSND [batch, s2, 1, d] | TND [T2, 1, d] | PA [blocks, block_size, 1, d] */
  const void* key_rope;   /* same with d_rope     */
  const int32_t* sparse_indices; /* [rows, 1, sparse_count] */
  const int32_t* seq_q;
  const int32_t* seq_k;
  const int32_t* block_table;
  void* out;              /* [rows, n1, d], dtype */
  float* softmax_max;     /* [rows, n1] (BSND view [batch,1,s1,n1], TND view [1,T1,n1]); NULL if !return_lse */
  float* softmax_sum;
  int32_t layout_q, layout_kv, dtype;
  int32_t seq_q_cumulative, seq_k_cumulative;
  int32_t batch, s1, s2, n1, d, d_rope;
  int32_t block_size, max_blocks;
  int32_t sparse_count, sparse_block_size, sparse_mode, return_lse;
  float scale;
  int64_t key_rows;     /* rows of the key tensor: batch*s2 (BSND), T2 (TND), blocks*block_size (PA) */
} DsaSfaParams;

/* Workspace size for dsa_li_forward (fp32 score rows + a status word). 256-byte aligned use. */
int dsa_li_workspace_bytes(const DsaLiParams* p, size_t* out_bytes);
/* Enqueue the indexer on `stream` (a cudaStream_t passed as void*). */
int dsa_li_forward(const DsaLiParams* p, void* workspace, size_t workspace_bytes, void* stream);

int dsa_sfa_workspace_bytes(const DsaSfaParams* p, size_t* out_bytes);
int dsa_sfa_forward(const DsaSfaParams* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * sparse_flash_attention backward - replaces `_sfa_grad_core`
 * (sparse_flash_attention_grad_triton.py:385-493) behind `sparse_flash_attention_grad_triton`
 * (:499-680).  Inputs are the forward operands, the gradient of the attention output, the
 * forward output and its softmax statistics; the five gradients have the shapes and dtype of
 * query, key, value (= key), query_rope, key_rope.  d_key holds the QK path and d_value the
 * PV path separately, as in the reference (a caller that shares key and value adds them).
 * Layouts BSND and TND (query and key/value); paged caches are not differentiated, as in the
 * reference.  The scatter-add over keys uses fp32 atomics in the workspace, so the last place
 * of d_key / d_value / d_key_rope can vary between runs (the reference refuses
 * deterministic=True for the same reason, :558-559).
 */
typedef struct DsaSfaGradParams {
  uint32_t struct_size; /* sizeof(DsaSfaGradParams) */
  int32_t kernel;       /* DSA_KERNEL_AUTO / _TENSOR: mma.sync kernel; _PORTABLE: CUDA-core kernel */
  const void* query;      /* [rows, n1, d]      */
  const void* query_rope; /* [rows, n1, d_rope] */
  const void* key;        /* BSND [batch, s2, 1, d] | TND [T2, 1, d] */
  const void* key_rope;
  const int32_t* sparse_indices; /* [rows, 1, sparse_count] */
  const void* d_out;      /* [rows, n1, d] */
  const void* out;        /* [rows, n1, d] */
  const float* softmax_max; /* [rows, n1] (BSND view [batch,1,s1,n1], TND view [1,T1,n1]) */
  const float* softmax_sum;
  const int32_t* seq_q;
  const int32_t* seq_k;
  void* d_query;      /* [rows, n1, d]      */
  void* d_query_rope; /* [rows, n1, d_rope] */
  void* d_key;        /* [key_rows, d]      */
  void* d_key_rope;   /* [key_rows, d_rope] */
  void* d_value;      /* [key_rows, d]      */
  int32_t layout_q, layout_kv, dtype;
  int32_t seq_q_cumulative, seq_k_cumulative;
  int32_t batch, s1, s2, n1, d, d_rope;
  int32_t sparse_count, sparse_block_size, sparse_mode;
  float scale;
  int64_t key_rows; /* batch*s2 (BSND) or T2 (TND) */
} DsaSfaGradParams;

/* Workspace: a status header plus fp32 accumulators key_rows * (2*d + d_rope) * 4 bytes. */
int dsa_sfa_grad_workspace_bytes(const DsaSfaGradParams* p, size_t* out_bytes);
/* Enqueue the backward on `stream`: clears the accumulators, runs the gradient kernel and the
 * conversion of the accumulators to the io dtype. */
int dsa_sfa_grad(const DsaSfaGradParams* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Backward of the sparse lightning indexer under the KL loss against the attention distribution -
 * replaces `_sparse_lightning_indexer_grad_kl_loss_core`
 * (sparse_lightning_indexer_grad_kl_loss_triton.py:331-443) behind
 * `sparse_lightning_indexer_grad_kl_loss_triton` (:496-580).  BSND, rightDownCausal, one key head.
 * Inputs: the attention operands (query / key with optional 64-wide rope parts), the indexer
 * operands (query_index, key_index, weights), the sparse indices and the softmax statistics of the
 * dense causal attention forward.  Outputs: d_query_index, d_key_index (dtype of the index tensors),
 * d_weights (dtype of weights) and the fp32 loss (one element).  d_key_index is a scatter-add with
 * fp32 atomics: its last place can vary between runs.
 *
 * With dense = 1 the same entry point is the dense operator, replacing
 * `_dense_loss_backward_with_index_core` / `_dense_loss_backward_core`
 * (dense_loss_backward_triton.py:423-598) behind `dense_loss_backward_triton` (:708-770): every
 * causally visible key takes part (sparse_indices is ignored and may be NULL, topk is ignored), the
 * attention key may have n2 heads (key [batch, s2, n2, d], statistics [batch, n2, s1, n1 / n2]) and
 * the student distribution is normalised with softmax_max_index / softmax_sum_index ([batch * s1]
 * fp32, as dsa_dense_li_lse produces them); when those are NULL they are computed internally.
 */
typedef struct DsaSliGradParams {
  uint32_t struct_size; /* sizeof(DsaSliGradParams) */
  int32_t kernel;       /* DSA_KERNEL_AUTO or DSA_KERNEL_PORTABLE (one implementation: both run it) */
  const void* query;       /* [batch, s1, n1, d]      */
  const void* query_rope;  /* [batch, s1, n1, d_rope] or NULL with d_rope = 0 */
  const void* key;         /* [batch, s2, 1, d]       */
  const void* key_rope;    /* [batch, s2, 1, d_rope] or NULL */
  const void* query_index; /* [batch, s1, g, d_idx]   */
  const void* key_index;   /* [batch, s2, 1, d_idx]   */
  const void* weights;     /* [batch, s1, g], dtype_w */
  const int32_t* sparse_indices; /* [batch, s1, 1, topk] */
  const float* softmax_max;      /* [batch, 1, s1, n1] */
  const float* softmax_sum;
  const int32_t* seq_q; /* [batch] valid query lengths or NULL */
  const int32_t* seq_k; /* [batch] valid key lengths or NULL   */
  void* d_query_index;  /* [batch, s1, g, d_idx] */
  void* d_key_index;    /* [batch, s2, 1, d_idx] */
  void* d_weights;      /* [batch, s1, g], dtype_w */
  float* loss;          /* [1] */
  int32_t dtype, dtype_w;
  int32_t batch, s1, s2, n1, d, d_rope, g, d_idx, topk;
  float scale;
  int32_t dense;                  /* 0: sparse operator, 1: dense operator */
  int32_t n2;                     /* attention key heads (1 for the sparse operator) */
  const float* softmax_max_index; /* dense: [batch * s1] or NULL */
  const float* softmax_sum_index;
} DsaSliGradParams;

/* Workspace: status header + fp32 scratch (index scores / dI and attention probabilities, each
 * [rows, slots]; one loss term per row; the d_key_index accumulator [batch * s2, d_idx]). */
int dsa_sli_grad_workspace_bytes(const DsaSliGradParams* p, size_t* out_bytes);
int dsa_sli_grad(const DsaSliGradParams* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Dense lightning-indexer softmax statistics - replaces `_dense_index_stats_core`
 * (dense_loss_backward_triton.py:344-420) behind `npu_dense_lightning_indexer_softmax_lse_triton`
 * (:773-802): per query row the maximum and the sum of exponentials over the causally visible keys
 * of I[k] = sum_g w[g] relu(query_index[g] . key_index[k]); -inf / 0 for rows that see no key.
 * Workspace: status header + the fp32 index scores [batch * s1, round_up(s2, 4)].  Shapes the
 * tensor-core scoring kernel of dsa_li_forward takes (16..64 index heads, d_idx 128) run it, followed
 * by one reduction per row; other shapes run CUDA-core kernels.
 */
typedef struct DsaDenseLseParams {
  uint32_t struct_size; /* sizeof(DsaDenseLseParams) */
  int32_t reserved;
  const void* query_index; /* [batch, s1, g, d_idx] */
  const void* key_index;   /* [batch, s2, 1, d_idx] */
  const void* weights;     /* [batch, s1, g], dtype_w */
  const int32_t* seq_q;    /* [batch] or NULL */
  const int32_t* seq_k;
  float* softmax_max_index; /* [batch * s1] */
  float* softmax_sum_index;
  int32_t dtype, dtype_w;
  int32_t batch, s1, s2, g, d_idx;
} DsaDenseLseParams;
int dsa_dense_li_lse_workspace_bytes(const DsaDenseLseParams* p, size_t* out_bytes);
int dsa_dense_li_lse(const DsaDenseLseParams* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * dsa_li_forward_static - the indexer without a caller workspace and without any allocation.
 * (No counterpart in the reference; added for hosts described below.)
 *
 * Some hosts of this operator cannot give it scratch memory: a graph-op boundary like the
 * reference's `_ms_pyfunc` core hands the kernel launcher exactly the tensors its shape
 * inference declared, and a launcher running inside such a callback must not call cudaMalloc
 * either - that would bypass the framework's memory pool, can fail once a serving engine has
 * reserved all of HBM for its caches, and synchronises the device.  For them the fp32 score
 * rows (the only scratch the indexer needs) live in a fixed array of
 * dsa_li_static_scratch_bytes() = 32 MiB inside the library image; every GPU that loads the
 * library holds that array until the process exits.
 *
 *  - Same parameters, results and status codes as dsa_li_forward with the portable kernels
 *    (kernel = DSA_KERNEL_AUTO or DSA_KERNEL_PORTABLE; DSA_KERNEL_TENSOR is refused with
 *    DSA_ERR_UNSUPPORTED).  The caller still passes every input and output buffer.
 *  - rows * n2 * round_up(s2, 4) * 4 bytes must fit the array, otherwise DSA_ERR_TOO_LARGE
 *    (e.g. 1024 query rows x 8192 keys, or 128 rows x 65536 keys).
 *  - It calls no cudaMalloc / cudaFree or other allocating routine.  The first call on each
 *    device looks up the array's device address (with that device current); make that first
 *    call outside any stream capture.
 *  - All calls on a device share the one array: calls whose kernels may overlap on the GPU
 *    (different streams, or different threads) race on it and must be serialised by the
 *    caller.  Nothing in the array needs to survive between calls.
 */
int dsa_li_forward_static(const DsaLiParams* p, void* stream);
size_t dsa_li_static_scratch_bytes(void);

/* Static description of a status code. */
const char* dsa_status_string(int status);
/* Synchronises `stream` and returns the device status word stored at the start of a
 * workspace: DSA_OK, or DSA_ERR_DEVICE_WAIT when a bounded in-kernel wait gave up. */
int dsa_read_device_status(const void* workspace, void* stream);
/* Self-test of the failure path (no counterpart in the reference, which reports nothing from the
 * device): enqueues a one-thread kernel that waits, with a limit of about half a millisecond, on a
 * barrier nothing ever signals, gives up and leaves the status word set - exactly what a tensor-core
 * kernel does when one of its bounded waits runs out.  dsa_read_device_status(workspace) then
 * returns DSA_ERR_DEVICE_WAIT; the device context stays usable.  `workspace`: >= 256 bytes,
 * 256-byte aligned. */
int dsa_selftest_wait_timeout(void* workspace, size_t workspace_bytes, void* stream);
/* 1 when dsa_*_forward would take the tcgen05 path for these parameters, else 0. */
int dsa_li_uses_tensor_path(const DsaLiParams* p);
int dsa_sfa_uses_tensor_path(const DsaSfaParams* p);
/* Number of CUDA kernels this library has launched in this process so far (all devices, all
 * entry points; memsets are not kernels).  No counterpart in the reference. */
unsigned long long dsa_kernel_launch_count(void);
/* ABI version of this header. */
int dsa_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DSA_B200_H_ */
