"""Domain parallelism: ``ShardTensor`` and the peer-memory collectives.

Parity: ``physicsnemo/domain_parallel`` (``ShardTensor``, ``ShardTensorSpec``, ``scatter_tensor``,
``sync_module_over_mesh``, ``TensorPromotionMode``).  ``physicsnemo_b200.domain_parallel`` is an
alias of this package.
"""
from torch.distributed.tensor import Partial, Replicate, Shard

from .grad_ops import defer_param_grad_reduction, reduce_param_grads
from .shard_tensor import MissingShardPatch, ShardTensor, TensorPromotionMode, scatter_tensor
from .spec import ShardTensorSpec
from .sync import sync_module_over_mesh

__all__ = [
    "ShardTensor", "ShardTensorSpec", "scatter_tensor", "sync_module_over_mesh", "TensorPromotionMode",
    "MissingShardPatch", "Shard", "Replicate", "Partial", "defer_param_grad_reduction", "reduce_param_grads",
]
