"""``ShardTensor``: a tensor distributed over a device mesh with uneven shards allowed.

Parity: ``physicsnemo/domain_parallel/shard_tensor.py`` — public API ``from_local``,
``redistribute``, ``to_local``, ``full_tensor``, ``backward``, ``offsets``, properties
``device_mesh / placements / grad``, handler registries (``register_function_handler``,
``register_dispatch_handler``, ``register_named_function_handler``), promotion modes, and
``scatter_tensor`` (``:1633-1756``).

Design (differs from the reference, which subclasses DTensor and intercepts aten ops):
``ShardTensor`` is a metadata wrapper.  Its ``shape`` is the *global* shape; the data and
the autograd graph live in the local shard, an ordinary ``torch.Tensor``.  Every
``torch`` / ``torch.nn.functional`` call that receives a ShardTensor arrives in
``__torch_function__`` and is resolved, in order, by

1. a registered handler (convolutions with halo exchange, normalisations with global
   statistics, ring attention, reductions, views, ... — ``physicsnemo_b200.parallel.patches``),
2. the generic *local rule* for operations that act independently on the unsharded
   dimensions (point-wise math, ``linear``, ``layer_norm`` over feature dims, ...),
3. ``MissingShardPatch``.

Communication happens only inside differentiable collectives on the local shards
(``collectives.py``), so model code runs unmodified and backward needs no extra machinery.
"""
from __future__ import annotations

import enum
import warnings
from typing import Callable, Dict, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import Partial, Replicate, Shard

from . import collectives as C
from .spec import ShardTensorSpec, chunk_sizes, infer_spec_from_local, mesh_coordinate


class MissingShardPatch(NotImplementedError):
    """Raised when an operation has no rule for the given sharding."""


class TensorPromotionMode(enum.Enum):
    """What to do when a plain tensor meets a ShardTensor in one operation."""

    DISABLED = "disabled"  # raise
    WARN = "warn"          # treat the plain tensor as replicated and warn once per op
    SILENT = "silent"      # treat the plain tensor as replicated


_NO_TF = torch._C.DisableTorchFunctionSubclass


class ShardTensor(torch.Tensor):
    _local_tensor: torch.Tensor
    _spec: ShardTensorSpec

    _function_registry: Dict[Callable, Callable] = {}
    _named_function_registry: Dict[str, Callable] = {}
    _dispatch_registry: Dict[object, Callable] = {}
    _promotion_mode = TensorPromotionMode.SILENT
    _warned: set = set()

    # ------------------------------------------------------------ creation
    @staticmethod
    def __new__(cls, local_tensor: torch.Tensor, spec: ShardTensorSpec):
        with _NO_TF():
            r = torch.Tensor._make_wrapper_subclass(
                cls, spec.global_shape, dtype=local_tensor.dtype, device=local_tensor.device,
                layout=local_tensor.layout, requires_grad=False)
        r._local_tensor = local_tensor
        r._spec = spec
        return r

    def __init__(self, *args, **kwargs):
        pass

    def __repr__(self):
        return (f"ShardTensor(local_shape={tuple(self._local_tensor.shape)}, global_shape={tuple(self._spec.global_shape)}, "
                f"placements={self._spec.placements}, mesh={tuple(self._spec.mesh.mesh.shape)})")

    # ----------------------------------------------------------- registries
    @classmethod
    def register_function_handler(cls, func: Callable, handler: Callable) -> None:
        """``handler(func, types, args, kwargs)`` takes over ``func`` for ShardTensor inputs."""
        cls._function_registry[func] = handler

    @classmethod
    def register_named_function_handler(cls, name: str, handler: Callable) -> None:
        cls._named_function_registry[name] = handler

    @classmethod
    def register_dispatch_handler(cls, op, handler: Callable) -> None:
        cls._dispatch_registry[op] = handler

    @classmethod
    def set_promotion_mode(cls, mode: TensorPromotionMode) -> None:
        cls._promotion_mode = TensorPromotionMode(mode)

    @classmethod
    def promotion_mode(cls) -> TensorPromotionMode:
        return cls._promotion_mode

    # ------------------------------------------------------------ properties
    @property
    def device_mesh(self) -> DeviceMesh:
        return self._spec.mesh

    @property
    def placements(self) -> Tuple:
        return self._spec.placements

    @property
    def spec(self) -> ShardTensorSpec:
        return self._spec

    @property
    def local_shape(self):
        return self._local_tensor.shape

    def offsets(self, mesh_dim: Optional[int] = None):
        return self._spec.offsets(mesh_dim)

    @property
    def requires_grad(self):
        return self._local_tensor.requires_grad

    @requires_grad.setter
    def requires_grad(self, value):
        self._local_tensor.requires_grad_(value)

    def requires_grad_(self, requires_grad: bool = True):
        self._local_tensor.requires_grad_(requires_grad)
        return self

    @property
    def grad(self):
        g = self._local_tensor.grad
        return None if g is None else ShardTensor(g, self._spec)

    @grad.setter
    def grad(self, value):
        self._local_tensor.grad = value._local_tensor if isinstance(value, ShardTensor) else value

    @property
    def grad_fn(self):
        return self._local_tensor.grad_fn

    @property
    def is_leaf(self):
        return self._local_tensor.is_leaf

    def detach(self):
        return ShardTensor(self._local_tensor.detach(), self._spec)

    def retain_grad(self):
        self._local_tensor.retain_grad()

    def register_hook(self, hook):
        return self._local_tensor.register_hook(hook)

    # --------------------------------------------------------- construction
    @staticmethod
    def from_local(local_tensor: torch.Tensor, device_mesh: Optional[DeviceMesh] = None,
                   placements: Optional[Sequence] = None, sharding_shapes="infer",
                   global_shape: Optional[Sequence[int]] = None) -> "ShardTensor":
        """Wrap this rank's shard. ``sharding_shapes``: ``"infer"`` (all-gather of extents),
        ``"chunk"`` (even split of ``global_shape``) or ``{mesh_dim: per-rank shapes}``."""
        if device_mesh is None:
            from ..distributed import DistributedManager

            device_mesh = DistributedManager().global_mesh
        if placements is None:
            placements = [Replicate()] * device_mesh.ndim
        spec = infer_spec_from_local(local_tensor, device_mesh, placements, sharding_shapes, global_shape)
        return ShardTensor(local_tensor, spec)

    def to_local(self, grad_placements=None) -> torch.Tensor:
        return self._local_tensor

    def full_tensor(self, grad_placements=None) -> torch.Tensor:
        """The global tensor on every rank (resolves Partial, gathers shards)."""
        return self.redistribute(placements=[Replicate()] * self._spec.mesh.ndim)._local_tensor

    def redistribute(self, device_mesh: Optional[DeviceMesh] = None, placements: Optional[Sequence] = None,
                     async_op: bool = False) -> "ShardTensor":
        from .redistribute import redistribute_shard_tensor

        if device_mesh is not None and device_mesh is not self._spec.mesh and device_mesh != self._spec.mesh:
            raise NotImplementedError("redistribution across different meshes is not supported")
        if placements is None:
            raise ValueError("placements are required")
        return redistribute_shard_tensor(self, tuple(placements))

    def backward(self, gradient=None, retain_graph=None, create_graph=False, inputs=None):
        """Backward from this tensor.  A Partial tensor stands for the sum of the ranks' values,
        so each rank seeds its own share; a replicated scalar is seeded with ``1/mesh_size`` so
        that the shares again add up to one."""
        local = self._local_tensor
        if isinstance(gradient, ShardTensor):
            gradient = gradient._local_tensor
        if gradient is None and self._spec.is_replicated() and local.numel() == 1:
            gradient = torch.full_like(local, 1.0 / self._spec.mesh.size())
        local.backward(gradient, retain_graph=retain_graph, create_graph=create_graph, inputs=inputs)

    def item(self):
        return self.full_tensor().item()

    def tolist(self):
        return self.full_tensor().tolist()

    def numpy(self):
        return self.full_tensor().detach().cpu().numpy()

    # -------------------------------------------------------------- dispatch
    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        from . import patches  # noqa: F401  (registers handlers on first use)
        from .local_rule import apply_local_rule, passthrough

        handler = cls._function_registry.get(func)
        if handler is None:
            name = getattr(func, "__name__", None)
            handler = cls._named_function_registry.get(name) if name else None
            qual = f"{getattr(func, '__module__', '')}.{name}"
            handler = handler or cls._named_function_registry.get(qual)
        if handler is not None:
            return handler(func, types, args, kwargs)
        hit, out = passthrough(func, args, kwargs)
        if hit:
            return out
        return apply_local_rule(func, args, kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        handler = cls._dispatch_registry.get(func)
        if handler is not None:
            return handler(func, types, args, kwargs or {})
        raise MissingShardPatch(
            f"aten op {func} reached ShardTensor dispatch without a handler; the calling torch function "
            "needs a ShardTensor rule (register one with ShardTensor.register_function_handler)"
        )


def scatter_tensor(tensor: Optional[torch.Tensor], global_src: int, mesh: DeviceMesh, placements: Sequence,
                   global_shape=None, dtype=None, requires_grad: bool = False) -> ShardTensor:
    """Distribute a tensor that exists on rank ``global_src`` over ``mesh`` with ``placements``.

    Shape / dtype are broadcast first; only the slab a rank needs is sent to it (point-to-point),
    instead of broadcasting the whole tensor and slicing (reference ``:1633-1756``).
    """
    from ..distributed import DistributedManager

    rank = dist.get_rank()
    meta = [None]
    if rank == global_src:
        if tensor is None:
            raise ValueError("the source rank must provide the tensor")
        meta[0] = (tuple(tensor.shape), tensor.dtype)
    group = DistributedManager().get_mesh_group(mesh) if mesh.ndim > 1 else mesh.get_group()
    dist.broadcast_object_list(meta, src=global_src, group=group)
    shape, dt = meta[0]
    placements = tuple(placements)
    device = tensor.device if tensor is not None else DistributedManager().device
    mesh_ranks = mesh.mesh.flatten().tolist()
    sizes = {md: chunk_sizes(shape[p.dim], mesh.size(md)) for md, p in enumerate(placements) if isinstance(p, Shard)}

    def slab_of(coord):
        sl = [slice(None)] * len(shape)
        for md, p in enumerate(placements):
            if isinstance(p, Shard):
                start = sum(sizes[md][: coord[md]])
                sl[p.dim] = slice(start, start + sizes[md][coord[md]])
        return tuple(sl)

    import numpy as _np

    coords = {int(mesh.mesh[idx]): tuple(int(c) for c in idx) for idx in _np.ndindex(*mesh.mesh.shape)}
    my_coord = coords[rank]
    my_shape = [s for s in shape]
    for md, p in enumerate(placements):
        if isinstance(p, Shard):
            my_shape[p.dim] = sizes[md][my_coord[md]]
    if rank == global_src:
        local = None
        reqs = []
        for r in mesh_ranks:
            piece = tensor[slab_of(coords[r])].contiguous()
            if r == rank:
                local = piece.clone()
            else:
                reqs.append(dist.isend(piece, dst=r))
        for q in reqs:
            q.wait()
    else:
        local = torch.empty(my_shape, dtype=dt, device=device)
        dist.recv(local, src=global_src)
    local.requires_grad_(requires_grad)
    spec = ShardTensorSpec(mesh=mesh, placements=placements, global_shape=torch.Size(shape), dtype=dt,
                           sharding_sizes=sizes)
    return ShardTensor(local, spec)
