"""Dense lightning-indexer softmax statistics and KL-loss backward on B200: the reference's public
operators, unchanged signatures.

Mirrors dense_loss_backward_triton.py:708-964: `dense_loss_backward_triton`,
`npu_dense_lightning_indexer_softmax_lse_triton` / `dense_lightning_indexer_softmax_lse_triton`,
`dense_lightning_indexer_grad_kl_loss_triton` / `npu_dense_lightning_indexer_grad_kl_loss_triton` and
the three Cells, with the reference's argument checks (:599-705).  BSND, sparse_mode 3; the attention
key may have N2 heads, the index key has one.
"""
import ctypes

import torch

from . import _cabi
from ._host import INT64_MAX, current_stream, dtype_code, note_launch, ptr, require_cuda, seq_tensor, workspace

SUPPORTED_D = (128, 256, 512)


def _validate_index_inputs(query_index, key_index, weights, layout, sparse_mode, pre_tokens, next_tokens):
    """dense_loss_backward_triton.py:599-625 (index head count: any, not only 32/64/128)."""
    if layout != "BSND":
        raise ValueError("Only BSND layout is supported")
    if sparse_mode != 3:
        raise ValueError("Only sparse_mode=3 (rightDownCausal) is supported")
    if pre_tokens != INT64_MAX or next_tokens != INT64_MAX:
        raise ValueError("pre_tokens/next_tokens only support the official default value")
    if query_index.ndim != 4 or key_index.ndim != 4:
        raise ValueError("query_index and key_index must be 4D BSND tensors")
    if weights.ndim != 3:
        raise ValueError("weights must be [B, S1, Nidx1]")
    B, S1, G, Di = query_index.shape
    if key_index.shape[0] != B or key_index.shape[2] != 1:
        raise ValueError("key_index must be [B, S2, 1, D_idx]")
    if tuple(weights.shape) != (B, S1, G):
        raise ValueError("weights must be [B, S1, Nidx1]")
    if key_index.shape[3] != Di:
        raise ValueError("query_index and key_index must share D_idx")
    if Di not in SUPPORTED_D:
        raise ValueError(f"D_idx must be one of {SUPPORTED_D}, got {Di}")
    if query_index.dtype not in (torch.float16, torch.bfloat16) or key_index.dtype != query_index.dtype:
        raise TypeError("query_index and key_index must share a float16 or bfloat16 dtype")
    if weights.dtype != query_index.dtype and weights.dtype != torch.float32:
        raise TypeError("weights dtype must match query dtype or be float32")


def npu_dense_lightning_indexer_softmax_lse_triton(query_index, key_index, weights, actual_seq_qlen=None,
                                                   actual_seq_klen=None, layout: str = "BSND", sparse_mode: int = 3,
                                                   pre_tokens: int = INT64_MAX, next_tokens: int = INT64_MAX):
    """Maximum and sum of exponentials, over the causally visible keys of every query row, of the
    indexer score I[k] = sum_g w[g] relu(query_index[g] . key_index[k]).

    Returns (softmax_max_index, softmax_sum_index), fp32 [B, 1, S1]; -inf / 0 where a row sees no key."""
    _validate_index_inputs(query_index, key_index, weights, layout, sparse_mode, pre_tokens, next_tokens)
    require_cuda(query_index, key_index, weights)
    dev = query_index.device
    B, S1, G, Di = query_index.shape
    S2 = key_index.shape[1]
    query_index, key_index, weights = query_index.contiguous(), key_index.contiguous(), weights.contiguous()
    seq_q, _ = seq_tensor(actual_seq_qlen, dev)
    seq_k, _ = seq_tensor(actual_seq_klen, dev)
    mx = torch.empty(B, 1, S1, dtype=torch.float32, device=dev)
    sm = torch.empty(B, 1, S1, dtype=torch.float32, device=dev)
    p = _cabi.DsaDenseLseParams()
    p.struct_size = ctypes.sizeof(_cabi.DsaDenseLseParams)
    p.query_index, p.key_index, p.weights = ptr(query_index), ptr(key_index), ptr(weights)
    p.seq_q, p.seq_k = ptr(seq_q), ptr(seq_k)
    p.softmax_max_index, p.softmax_sum_index = ptr(mx), ptr(sm)
    p.dtype = dtype_code(query_index, (torch.bfloat16, torch.float16), "query_index")
    p.dtype_w = dtype_code(weights, (torch.bfloat16, torch.float16, torch.float32), "weights")
    p.batch, p.s1, p.s2, p.g, p.d_idx = B, S1, S2, G, Di
    with torch.cuda.device(dev):
        nbytes = ctypes.c_size_t(0)
        _cabi.check(_cabi.lib.dsa_dense_li_lse_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)),
                    "dense_lightning_indexer_softmax_lse")
        ws = workspace(nbytes.value, dev)
        _cabi.check(_cabi.lib.dsa_dense_li_lse(ctypes.byref(p), ws.data_ptr(), ws.numel(), current_stream(dev)),
                    "dense_lightning_indexer_softmax_lse")
        note_launch("dense_lightning_indexer_softmax_lse", ws, dev)
    return mx, sm


dense_lightning_indexer_softmax_lse_triton = npu_dense_lightning_indexer_softmax_lse_triton


def _index_stat(stat, B, S1, name):
    """dense_loss_backward_triton.py:696-705: [B,S1], [B*S1], [B,1,S1] or [B,1,S1,1] -> [B*S1]."""
    if tuple(stat.shape) in ((B, S1), (B * S1,), (B, 1, S1), (B, 1, S1, 1)):
        return stat.reshape(B * S1).contiguous()
    raise ValueError(f"{name} must have shape [B,S1], [B*S1], [B,1,S1], or [B,1,S1,1], got {tuple(stat.shape)}")


def dense_loss_backward_triton(query, key, query_index, key_index, weights, softmax_max, softmax_sum,
                               softmax_max_index=None, softmax_sum_index=None, scale_value: float = 1.0,
                               query_rope=None, key_rope=None, actual_seq_qlen=None, actual_seq_klen=None,
                               layout: str = "BSND", sparse_mode: int = 3, pre_tokens: int = INT64_MAX,
                               next_tokens: int = INT64_MAX):
    """Dense lightning-indexer KL-loss backward: like the sparse operator, over every causally visible key.

    query [B,S1,N1,D], key [B,S2,N2,D] (N1 divisible by N2), optional 64-wide rope parts,
    query_index [B,S1,G,Di], key_index [B,S2,1,Di], weights [B,S1,G], softmax_max / softmax_sum fp32
    [B,N2,S1,N1/N2] of the attention forward, softmax_max_index / softmax_sum_index fp32 per query row
    (computed internally when both are omitted).

    Returns (d_query_index, d_key_index, d_weights, loss[1])."""
    if query.ndim != 4 or key.ndim != 4:
        raise ValueError("query and key must be 4D BSND tensors")
    _validate_index_inputs(query_index, key_index, weights, layout, sparse_mode, pre_tokens, next_tokens)
    if query.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"query dtype must be float16 or bfloat16, got {query.dtype}")
    if key.dtype != query.dtype or query_index.dtype != query.dtype:
        raise TypeError("query, key, query_index, and key_index must share dtype")
    if softmax_max.dtype != torch.float32 or softmax_sum.dtype != torch.float32:
        raise TypeError("softmax_max and softmax_sum must be float32")
    B, S1, N1, D = query.shape
    if key.shape[0] != B or key.shape[3] != D:
        raise ValueError("key must be [B, S2, N2, D_attn]")
    S2, N2 = key.shape[1], key.shape[2]
    if N2 <= 0 or N1 % N2 != 0:
        raise ValueError("query N1 must be divisible by key N2")
    if query_index.shape[0] != B or query_index.shape[1] != S1:
        raise ValueError("query_index must share B and S1 with query")
    if key_index.shape[1] != S2:
        raise ValueError("key_index S2 must match key S2")
    stat_shape = (B, N2, S1, N1 // N2)
    if tuple(softmax_max.shape) != stat_shape or tuple(softmax_sum.shape) != stat_shape:
        raise ValueError(f"softmax_max and softmax_sum must be [B, N2, S1, G], got {tuple(softmax_max.shape)}")
    if D not in SUPPORTED_D:
        raise ValueError(f"D_attn must be one of {SUPPORTED_D}, got {D}")
    if (query_rope is None) != (key_rope is None):
        raise ValueError("query_rope and key_rope must be both provided or both omitted")
    d_rope = 0
    if query_rope is not None:
        if query_rope.ndim != 4 or key_rope.ndim != 4:
            raise ValueError("query_rope and key_rope must be 4D BSND tensors")
        if tuple(query_rope.shape[:3]) != (B, S1, N1) or tuple(key_rope.shape[:3]) != (B, S2, N2):
            raise ValueError("rope parts must share [B, S, N] with query / key")
        if query_rope.shape[3] != 64 or key_rope.shape[3] != 64:
            raise ValueError("Only Drope=64 is supported for query_rope/key_rope")
        if query_rope.dtype != query.dtype or key_rope.dtype != key.dtype:
            raise TypeError("query_rope/key_rope dtype must match query/key dtype")
        d_rope = 64
    if (softmax_max_index is None) != (softmax_sum_index is None):
        raise ValueError("softmax_max_index and softmax_sum_index must be both provided or both omitted")
    if softmax_max_index is not None:
        if softmax_max_index.dtype != torch.float32 or softmax_sum_index.dtype != torch.float32:
            raise TypeError("softmax_max_index and softmax_sum_index must be float32")
        softmax_max_index = _index_stat(softmax_max_index, B, S1, "softmax_max_index")
        softmax_sum_index = _index_stat(softmax_sum_index, B, S1, "softmax_sum_index")
    require_cuda(query, key, query_index, key_index, weights, softmax_max, softmax_sum, softmax_max_index,
                 softmax_sum_index, query_rope, key_rope)
    dev = query.device

    query, key = query.contiguous(), key.contiguous()
    query_index, key_index, weights = query_index.contiguous(), key_index.contiguous(), weights.contiguous()
    softmax_max, softmax_sum = softmax_max.contiguous(), softmax_sum.contiguous()
    if d_rope:
        query_rope, key_rope = query_rope.contiguous(), key_rope.contiguous()
    seq_q, _ = seq_tensor(actual_seq_qlen, dev)
    seq_k, _ = seq_tensor(actual_seq_klen, dev)
    G, Di = query_index.shape[2], query_index.shape[3]

    d_query_index = torch.empty_like(query_index)
    d_key_index = torch.empty_like(key_index)
    d_weights = torch.empty_like(weights)
    loss = torch.empty(1, dtype=torch.float32, device=dev)

    p = _cabi.DsaSliGradParams()
    p.struct_size = ctypes.sizeof(_cabi.DsaSliGradParams)
    p.kernel = _cabi.KERNEL_AUTO
    p.query, p.query_rope, p.key, p.key_rope = ptr(query), ptr(query_rope), ptr(key), ptr(key_rope)
    p.query_index, p.key_index, p.weights = ptr(query_index), ptr(key_index), ptr(weights)
    p.softmax_max, p.softmax_sum = ptr(softmax_max), ptr(softmax_sum)
    p.seq_q, p.seq_k = ptr(seq_q), ptr(seq_k)
    p.d_query_index, p.d_key_index, p.d_weights, p.loss = ptr(d_query_index), ptr(d_key_index), ptr(d_weights), ptr(loss)
    p.dtype = dtype_code(query, (torch.bfloat16, torch.float16), "query")
    p.dtype_w = dtype_code(weights, (torch.bfloat16, torch.float16, torch.float32), "weights")
    p.batch, p.s1, p.s2, p.n1, p.d, p.d_rope = B, S1, S2, N1, D, d_rope
    p.g, p.d_idx, p.topk = G, Di, 0
    p.scale = float(scale_value)
    p.dense, p.n2 = 1, N2
    p.softmax_max_index, p.softmax_sum_index = ptr(softmax_max_index), ptr(softmax_sum_index)

    with torch.cuda.device(dev):
        nbytes = ctypes.c_size_t(0)
        _cabi.check(_cabi.lib.dsa_sli_grad_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)), "dense_loss_backward")
        ws = workspace(nbytes.value, dev)
        _cabi.check(_cabi.lib.dsa_sli_grad(ctypes.byref(p), ws.data_ptr(), ws.numel(), current_stream(dev)),
                    "dense_loss_backward")
        note_launch("dense_loss_backward", ws, dev)
    return d_query_index, d_key_index, d_weights, loss


def dense_lightning_indexer_grad_kl_loss_triton(query, key, query_index, key_index, weights, softmax_max, softmax_sum,
                                                softmax_max_index, softmax_sum_index, scale_value, query_rope=None,
                                                key_rope=None, actual_seq_qlen=None, actual_seq_klen=None,
                                                layout: str = "BSND", sparse_mode: int = 3,
                                                pre_tokens: int = INT64_MAX, next_tokens: int = INT64_MAX):
    """Official-style name of dense_loss_backward_triton (dense_loss_backward_triton.py:819-849)."""
    return dense_loss_backward_triton(
        query, key, query_index, key_index, weights, softmax_max, softmax_sum, softmax_max_index,
        softmax_sum_index, scale_value, query_rope=query_rope, key_rope=key_rope,
        actual_seq_qlen=actual_seq_qlen, actual_seq_klen=actual_seq_klen, layout=layout,
        sparse_mode=sparse_mode, pre_tokens=pre_tokens, next_tokens=next_tokens)


npu_dense_lightning_indexer_grad_kl_loss_triton = dense_lightning_indexer_grad_kl_loss_triton


class DenseLightningIndexerSoftmaxLseTriton(torch.nn.Module):
    """dense_loss_backward_triton.py:885-901."""

    def forward(self, query_index, key_index, weight, actual_seq_qlen=None, actual_seq_klen=None, layout="BSND",
                sparse_mode=3, pre_tokens=INT64_MAX, next_tokens=INT64_MAX):
        return npu_dense_lightning_indexer_softmax_lse_triton(
            query_index, key_index, weight, actual_seq_qlen=actual_seq_qlen, actual_seq_klen=actual_seq_klen,
            layout=layout, sparse_mode=sparse_mode, pre_tokens=pre_tokens, next_tokens=next_tokens)

    construct = forward


class DenseLossBackwardTriton(torch.nn.Module):
    """dense_loss_backward_triton.py:904-936."""

    def __init__(self, scale_value=1.0, layout="BSND", sparse_mode=3, pre_tokens=INT64_MAX, next_tokens=INT64_MAX):
        super().__init__()
        self.scale_value = scale_value
        self.layout = layout
        self.sparse_mode = sparse_mode
        self.pre_tokens = pre_tokens
        self.next_tokens = next_tokens

    def forward(self, query, key, query_index, key_index, weights, softmax_max, softmax_sum,
                softmax_max_index=None, softmax_sum_index=None, scale_value=None, query_rope=None, key_rope=None,
                actual_seq_qlen=None, actual_seq_klen=None):
        return dense_loss_backward_triton(
            query, key, query_index, key_index, weights, softmax_max, softmax_sum, softmax_max_index,
            softmax_sum_index, self.scale_value if scale_value is None else scale_value,
            query_rope=query_rope, key_rope=key_rope, actual_seq_qlen=actual_seq_qlen,
            actual_seq_klen=actual_seq_klen, layout=self.layout, sparse_mode=self.sparse_mode,
            pre_tokens=self.pre_tokens, next_tokens=self.next_tokens)

    construct = forward


class DenseLightningIndexerGradKLLossTriton(torch.nn.Module):
    """dense_loss_backward_triton.py:939-964."""

    def forward(self, query, key, query_index, key_index, weights, softmax_max, softmax_sum, softmax_max_index,
                softmax_sum_index, scale_value=1.0, query_rope=None, key_rope=None, actual_seq_qlen=None,
                actual_seq_klen=None, layout="BSND", sparse_mode=3, pre_tokens=INT64_MAX, next_tokens=INT64_MAX):
        return dense_loss_backward_triton(
            query, key, query_index, key_index, weights, softmax_max, softmax_sum, softmax_max_index,
            softmax_sum_index, scale_value, query_rope=query_rope, key_rope=key_rope,
            actual_seq_qlen=actual_seq_qlen, actual_seq_klen=actual_seq_klen, layout=layout,
            sparse_mode=sparse_mode, pre_tokens=pre_tokens, next_tokens=next_tokens)

    construct = forward
