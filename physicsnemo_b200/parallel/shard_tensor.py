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
        r._lt = local_tensor
        r._pending = None        # CUDA event of a redistribution issued with async_op=True on a side stream
        r._spec = spec
        return r

    @property
    def _local_tensor(self) -> torch.Tensor:
        """This rank's shard.  The first access after an asynchronous redistribution makes the current stream wait for
        the side stream that produced it."""
        ev = self._pending
        if ev is not None:
            torch.cuda.current_stream(self._lt.device).wait_event(ev)
            self._lt.record_stream(torch.cuda.current_stream(self._lt.device))
            self._pending = None
        return self._lt

    @_local_tensor.setter
    def _local_tensor(self, value: torch.Tensor) -> None:
        self._lt = value
        self._pending = None

    # -------------------------------------------------------- traceable wrapper-subclass protocol
    def __tensor_flatten__(self):
        """Inner tensors and the rest of the state (``torch.compile`` / AOT autograd wrapper-subclass protocol)."""
        return ["_local_tensor"], (self._spec,)

    @staticmethod
    def __tensor_unflatten__(inner_tensors, meta, outer_size=None, outer_stride=None):
        return ShardTensor(inner_tensors["_local_tensor"], meta[0])

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

    @staticmethod
    def from_dtensor(dtensor) -> "ShardTensor":
        """A ``torch.distributed.tensor.DTensor`` as a ShardTensor (no copy, no communication): DTensor shards are the
        ``torch.chunk`` pieces of the global tensor, which is the ``"chunk"`` rule of ``from_local``.  ``Partial``
        placements carry over.  Reference: ``ShardTensor.from_dtensor`` (``domain_parallel/shard_tensor.py:957-1005``)."""
        local = dtensor.to_local()
        return ShardTensor.from_local(local, dtensor.device_mesh, tuple(dtensor.placements), sharding_shapes="chunk",
                                      global_shape=tuple(dtensor.shape))

    def to_dtensor(self):
        """The same data as a DTensor; only for shardings a DTensor can express (``torch.chunk`` pieces)."""
        from torch.distributed.tensor import DTensor

        mesh, spec = self._spec.mesh, self._spec
        for md, p in enumerate(spec.placements):
            if isinstance(p, Shard):
                n = mesh.size(md)
                full = spec.global_shape[p.dim]
                even = [len(c) for c in torch.arange(full).chunk(n)] + [0] * n
                have = [int(v) for v in spec.sharding_sizes[md]]
                if have != even[:n]:
                    raise ValueError("uneven shards that are not torch.chunk pieces have no DTensor equivalent; redistribute first")
        return DTensor.from_local(self._local_tensor, mesh, tuple(spec.placements), run_check=False,
                                  shape=torch.Size(spec.global_shape), stride=torch.empty(spec.global_shape, device="meta").stride())

    def to_local(self, grad_placements=None) -> torch.Tensor:
        """This rank's shard (it carries the autograd graph itself).  ``grad_placements`` states how the gradient that
        later flows into the returned tensor is laid out over the mesh: ``Partial`` on a mesh dimension where this tensor
        is replicated means every rank will hold only a share of the gradient, so the shares are summed over that mesh
        dimension on the way back (reference: ``to_local(grad_placements=...)``, ``shard_tensor.py:1331``)."""
        local = self._local_tensor
        if grad_placements is None:
            return local
        from . import collectives as C

        grad_placements = tuple(grad_placements)
        if len(grad_placements) != self._spec.mesh.ndim:
            raise ValueError(f"grad_placements needs one entry per mesh dimension ({self._spec.mesh.ndim})")
        for md, (own, g) in enumerate(zip(self._spec.placements, grad_placements)):
            if isinstance(g, Partial) and isinstance(own, Replicate):
                local = C.GradAllReduce.apply(local, self._spec.mesh.get_group(md))
            elif type(g) is not type(own) or (isinstance(g, Shard) and g.dim != own.dim):
                raise NotImplementedError(f"gradient layout {g} for a tensor placed as {own} on mesh dimension {md}")
        return local

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
        local = self._local_tensor
        if not (async_op and local.is_cuda):
            return redistribute_shard_tensor(self, tuple(placements))
        # asynchronous: the collectives run on a side stream; the result waits for them at its first use
        cur = torch.cuda.current_stream(local.device)
        side = _side_stream(local.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            out = redistribute_shard_tensor(self, tuple(placements))
            ev = torch.cuda.Event()
            ev.record(side)
        local.record_stream(side)
        if out is not self:
            out._pending = ev
        return out

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


_side_streams: Dict[int, "torch.cuda.Stream"] = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _side_streams.get(key)
    if st is None:
        st = _side_streams[key] = torch.cuda.Stream(device=device)
    return st


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
