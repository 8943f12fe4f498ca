"""Backward of the sparse lightning indexer under the KL loss, on B200: the reference's public
operator, unchanged signature.

Mirrors `sparse_lightning_indexer_grad_kl_loss_triton` and
`SparseLightningIndexerGradKLLossTriton`
(sparse_lightning_indexer_grad_kl_loss_triton.py:446-580): same argument names and defaults, the
BSND / sparse_mode=3 guards, outputs (d_query_index, d_key_index, d_weights, loss[1]).  The
reference splits long query ranges into chunks of rows on the host and sums the pieces
(:520-580); the kernels here take any number of rows in one call.
"""
import ctypes

import torch

from . import _cabi
from ._host import INT64_MAX, current_stream, dtype_code, note_launch, ptr, require_cuda, seq_tensor, workspace


def sparse_lightning_indexer_grad_kl_loss_triton(
    query, key,
    query_index, key_index,
    weights, sparse_indices,
    softmax_max, softmax_sum,
    query_rope=None, key_rope=None,
    actual_seq_qlen=None, actual_seq_klen=None,
    scale_value: float = 1.0,
    layout: str = "BSND", sparse_mode: int = 3,
    pre_tokens: int = INT64_MAX,
    next_tokens: int = INT64_MAX,
    deterministic: bool = False,
):
    """Gradients of KL(attention distribution || softmax of the indexer scores) with respect to the
    indexer's inputs, over the keys the sparse indices select.

    Args (as sparse_lightning_indexer_grad_kl_loss_triton.py:496-509):
        query [B,S1,N1,D], key [B,S2,1,D]: attention operands, fp16/bf16, D in 128/256/512
        query_index [B,S1,G,Di], key_index [B,S2,1,Di]: indexer operands, Di in 128/256/512
        weights [B,S1,G]: indexer head weights (io dtype or fp32)
        sparse_indices [B,S1,1,topK] int32: selected key positions (clipped to [0, S2))
        softmax_max / softmax_sum [B,1,S1,N1] fp32: statistics of the dense causal attention forward
        query_rope / key_rope: optional 64-wide rope parts of the attention operands
        actual_seq_qlen / actual_seq_klen: [B] valid lengths or None
        scale_value: softmax scale of the attention scores
        layout "BSND" and sparse_mode 3 only; pre_tokens / next_tokens / deterministic are ignored
        like in the reference

    Returns:
        (d_query_index, d_key_index, d_weights, loss) - loss is fp32 of shape [1].
    """
    if layout != "BSND":
        raise ValueError("Only BSND layout is supported in triton path")
    if sparse_mode != 3:
        raise ValueError("Only sparse_mode=3 (rightDownCausal) is supported")
    if sparse_indices.shape[2] != 1:
        raise ValueError("Nidx2 must be 1 (MQA constraint)")
    if (query_rope is None) != (key_rope is None):
        raise ValueError("query_rope and key_rope must be given together")

    B, S1, N1, D = query.shape
    S2, N2 = key.shape[1], key.shape[2]
    G, Di = query_index.shape[2], query_index.shape[3]
    topk = sparse_indices.shape[3]
    d_rope = 0 if query_rope is None else query_rope.shape[-1]
    if N2 != 1 or key_index.shape[2] != 1:
        raise ValueError("Only one key head (MQA) is supported")
    if D not in (128, 256, 512) or Di not in (128, 256, 512):
        raise ValueError(f"head dims must be 128, 256 or 512, got D={D}, D_idx={Di}")
    if d_rope not in (0, 64):
        raise ValueError(f"rope dim must be 64, got {d_rope}")
    tensors = [query, key, query_index, key_index] + ([query_rope, key_rope] if d_rope else [])
    if any(t.dtype != query.dtype for t in tensors):
        raise ValueError("query, key, rope parts, query_index and key_index must share a dtype")
    stat_shape = (B, 1, S1, N1)
    if tuple(softmax_max.shape) != stat_shape or tuple(softmax_sum.shape) != stat_shape:
        raise ValueError(f"softmax_max / softmax_sum must have shape {stat_shape}")
    if tuple(weights.shape) != (B, S1, G) or key.shape[-1] != D or key_index.shape[-1] != Di:
        raise ValueError("weights / key / key_index shapes do not match the queries")
    require_cuda(query, key, query_index, key_index, weights, sparse_indices, softmax_max, softmax_sum,
                 query_rope, key_rope)
    dev = query.device

    query, key = query.contiguous(), key.contiguous()
    query_index, key_index, weights = query_index.contiguous(), key_index.contiguous(), weights.contiguous()
    if d_rope:
        query_rope, key_rope = query_rope.contiguous(), key_rope.contiguous()
    sparse_indices = sparse_indices.to(torch.int32).contiguous()
    softmax_max = softmax_max.to(torch.float32).contiguous()
    softmax_sum = softmax_sum.to(torch.float32).contiguous()
    seq_q, _ = seq_tensor(actual_seq_qlen, dev)
    seq_k, _ = seq_tensor(actual_seq_klen, dev)

    d_query_index = torch.empty_like(query_index)
    d_key_index = torch.empty_like(key_index)
    d_weights = torch.empty_like(weights)
    loss = torch.empty(1, dtype=torch.float32, device=dev)

    p = _cabi.DsaSliGradParams()
    p.struct_size = ctypes.sizeof(_cabi.DsaSliGradParams)
    p.kernel = _cabi.KERNEL_AUTO
    p.query, p.query_rope, p.key, p.key_rope = ptr(query), ptr(query_rope), ptr(key), ptr(key_rope)
    p.query_index, p.key_index, p.weights = ptr(query_index), ptr(key_index), ptr(weights)
    p.sparse_indices = ptr(sparse_indices)
    p.softmax_max, p.softmax_sum = ptr(softmax_max), ptr(softmax_sum)
    p.seq_q, p.seq_k = ptr(seq_q), ptr(seq_k)
    p.d_query_index, p.d_key_index, p.d_weights, p.loss = ptr(d_query_index), ptr(d_key_index), ptr(d_weights), ptr(loss)
    p.dtype = dtype_code(query, (torch.bfloat16, torch.float16), "query")
    p.dtype_w = dtype_code(weights, (torch.bfloat16, torch.float16, torch.float32), "weights")
    p.batch, p.s1, p.s2, p.n1, p.d, p.d_rope = B, S1, S2, N1, D, d_rope
    p.g, p.d_idx, p.topk = G, Di, topk
    p.scale = float(scale_value)

    with torch.cuda.device(dev):
        nbytes = ctypes.c_size_t(0)
        _cabi.check(_cabi.lib.dsa_sli_grad_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)),
                    "sparse_lightning_indexer_grad_kl_loss")
        ws = workspace(nbytes.value, dev)
        _cabi.check(_cabi.lib.dsa_sli_grad(ctypes.byref(p), ws.data_ptr(), ws.numel(), current_stream(dev)),
                    "sparse_lightning_indexer_grad_kl_loss")
        note_launch("sparse_lightning_indexer_grad_kl_loss", ws, dev)
    return d_query_index, d_key_index, d_weights, loss


class SparseLightningIndexerGradKLLossTriton(torch.nn.Module):
    """Attribute holder around sparse_lightning_indexer_grad_kl_loss_triton
    (sparse_lightning_indexer_grad_kl_loss_triton.py:446-493)."""

    def __init__(self, scale_value=1.0, layout="BSND", sparse_mode=3, pre_tokens=INT64_MAX,
                 next_tokens=INT64_MAX, deterministic=False):
        super().__init__()
        self.scale_value = scale_value
        self.layout = layout
        self.sparse_mode = sparse_mode
        self.pre_tokens = pre_tokens
        self.next_tokens = next_tokens
        self.deterministic = deterministic

    def forward(self, query, key, query_index, key_index, weights, sparse_indices, softmax_max, softmax_sum,
                query_rope=None, key_rope=None, actual_seq_qlen=None, actual_seq_klen=None):
        return sparse_lightning_indexer_grad_kl_loss_triton(
            query, key, query_index, key_index, weights, sparse_indices, softmax_max, softmax_sum,
            query_rope=query_rope, key_rope=key_rope,
            actual_seq_qlen=actual_seq_qlen, actual_seq_klen=actual_seq_klen,
            scale_value=self.scale_value, layout=self.layout, sparse_mode=self.sparse_mode,
            pre_tokens=self.pre_tokens, next_tokens=self.next_tokens, deterministic=self.deterministic)

    construct = forward
