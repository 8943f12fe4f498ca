"""B200-native (sm_100a) DeepSeek-Sparse-Attention hot path.

Public API = the operators of WhFanatic/dsa_triton_ascend with unchanged signatures:
`lightning_indexer_triton` / `LightningIndexerTriton`, `sparse_flash_attention_triton` /
`SparseFlashAttentionTriton`, the attention backward `sparse_flash_attention_grad_triton` /
`SparseFlashAttentionGradTriton` and the indexer's KL-loss backward
`sparse_lightning_indexer_grad_kl_loss_triton` / `SparseLightningIndexerGradKLLossTriton`, and the
dense counterpart with its statistics helper (`dense_loss_backward_triton`,
`dense_lightning_indexer_softmax_lse_triton`, ... in `dense_loss_backward`).  All are thin wrappers over the C-ABI CUDA library built from
`dsa_triton_ascend_b200/csrc` (declared in `include/dsa_b200.h`).  `check_status()` (an
addition) reports a device-side wait that ran out in the latest call of either operator.
"""
from ._host import check_status  # noqa: F401
from .lightning_indexer import LightningIndexerTriton, lightning_indexer_triton  # noqa: F401
from .sparse_flash_attention import SparseFlashAttentionTriton, sparse_flash_attention_triton  # noqa: F401
from .sparse_flash_attention_grad import (SparseFlashAttentionGradTriton,  # noqa: F401
                                          sparse_flash_attention_grad_triton)
from .sparse_lightning_indexer_grad_kl_loss import (SparseLightningIndexerGradKLLossTriton,  # noqa: F401
                                                     sparse_lightning_indexer_grad_kl_loss_triton)
from .dense_loss_backward import (DenseLightningIndexerGradKLLossTriton,  # noqa: F401
                                  DenseLightningIndexerSoftmaxLseTriton, DenseLossBackwardTriton,
                                  dense_lightning_indexer_grad_kl_loss_triton,
                                  dense_lightning_indexer_softmax_lse_triton, dense_loss_backward_triton,
                                  npu_dense_lightning_indexer_grad_kl_loss_triton,
                                  npu_dense_lightning_indexer_softmax_lse_triton)

__all__ = [
    "lightning_indexer_triton", "LightningIndexerTriton",
    "sparse_flash_attention_triton", "SparseFlashAttentionTriton",
    "sparse_flash_attention_grad_triton", "SparseFlashAttentionGradTriton",
    "sparse_lightning_indexer_grad_kl_loss_triton", "SparseLightningIndexerGradKLLossTriton",
    "dense_loss_backward_triton", "dense_lightning_indexer_softmax_lse_triton",
    "npu_dense_lightning_indexer_softmax_lse_triton", "dense_lightning_indexer_grad_kl_loss_triton",
    "npu_dense_lightning_indexer_grad_kl_loss_triton", "DenseLightningIndexerSoftmaxLseTriton",
    "DenseLossBackwardTriton", "DenseLightningIndexerGradKLLossTriton",
    "check_status",
]
