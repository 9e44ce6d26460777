"""Handlers that teach ``ShardTensor`` the operations needing more than the local rule.
Importing this package registers them (done lazily on the first ShardTensor operation)."""
from . import attention, conv, natten, neighbors, norm, reductions, spatial, view_ops  # noqa: F401
