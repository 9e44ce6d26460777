from .autograd import all_gather_v, gather_v, indexed_all_to_all_v, scatter_v
from .config import ProcessGroupConfig, ProcessGroupNode
from .fused_all_reduce import fused_all_reduce
from .manager import (
    DistributedManager,
    PhysicsNeMoUndefinedGroupError,
    PhysicsNeMoUninitializedDistributedManagerWarning,
)
from .utils import mark_module_as_shared, reduce_loss, unmark_module_as_shared

__all__ = [
    "DistributedManager", "PhysicsNeMoUndefinedGroupError", "PhysicsNeMoUninitializedDistributedManagerWarning",
    "ProcessGroupConfig", "ProcessGroupNode", "all_gather_v", "gather_v", "scatter_v", "indexed_all_to_all_v",
    "fused_all_reduce", "mark_module_as_shared", "unmark_module_as_shared", "reduce_loss",
]
