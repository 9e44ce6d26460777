"""Shape-only operations on ShardTensors (no communication).

Parity: ``physicsnemo/domain_parallel/shard_utils/view_ops.py`` (dimension-group matching that
carries a shard through ``view`` / ``reshape``), ``unary_ops.py`` (``unsqueeze``),
``custom_ops/_tensor_ops.py`` (``unbind``), ``index_ops.py`` (``select`` / ``__getitem__``).
"""
from __future__ import annotations

import math
from typing import List, Sequence

import torch
from torch.distributed.tensor import Partial, Replicate, Shard

from ._common import MissingShardPatch, NO_TF, ShardTensor, is_st, local, norm_dim, register, wrap


def _shape_arg(args, kwargs):
    if "shape" in kwargs:
        return list(kwargs["shape"])
    if "size" in kwargs:
        return list(kwargs["size"])
    rest = args[1:]
    if len(rest) == 1 and isinstance(rest[0], (list, tuple, torch.Size)):
        return list(rest[0])
    return list(rest)


def _match_groups(old: Sequence[int], new: Sequence[int]):
    """Split both shapes into minimal groups of dims with equal products: [(old_idx, new_idx), ...]."""
    groups, i, j = [], 0, 0
    while i < len(old) or j < len(new):
        oi, nj = [i] if i < len(old) else [], [j] if j < len(new) else []
        po = old[i] if i < len(old) else 1
        pn = new[j] if j < len(new) else 1
        i += 1 if i < len(old) else 0
        j += 1 if j < len(new) else 0
        while po != pn:
            if po < pn and i < len(old):
                po *= old[i]; oi.append(i); i += 1
            elif pn < po and j < len(new):
                pn *= new[j]; nj.append(j); j += 1
            else:
                raise MissingShardPatch(f"cannot match view {tuple(old)} -> {tuple(new)}")
        groups.append((oi, nj))
    # absorb trailing size-1 dims
    return groups


@register(torch.Tensor.reshape, torch.reshape, torch.Tensor.view, torch.Tensor.reshape_as, torch.Tensor.view_as)
def _reshape(func, types, args, kwargs):
    x: ShardTensor = args[0]
    if func in (torch.Tensor.reshape_as, torch.Tensor.view_as):
        new = list(args[1].shape)
    else:
        new = _shape_arg(args, kwargs)
    if len(new) == 1 and isinstance(new[0], torch.dtype):  # dtype view
        with NO_TF():
            out = local(x).view(new[0])
        return wrap(out, x._spec.mesh, x._spec.placements, x._spec.sharding_sizes)
    old = list(x.shape)
    if -1 in new:
        known = math.prod(s for s in new if s != -1)
        new[new.index(-1)] = math.prod(old) // max(known, 1)
    spec = x._spec
    sharded = {p.dim: md for md, p in enumerate(spec.placements) if isinstance(p, Shard)}
    if not sharded:
        with NO_TF():
            out = local(x).reshape(new)
        return wrap(out, spec.mesh, spec.placements, {})
    groups = _match_groups(old, new)
    local_new = list(new)
    placements = list(spec.placements)
    sizes = {}
    for oi, nj in groups:
        hit = [d for d in oi if d in sharded]
        if not hit:
            continue
        if len(hit) > 1:
            raise MissingShardPatch("two sharded dims merge into one in reshape")
        d = hit[0]
        md = sharded[d]
        # the sharded dim must be the leading (slowest) non-unit dim of its group on both sides
        lead_old = [k for k in oi if old[k] != 1]
        lead_new = [k for k in nj if new[k] != 1]
        if (lead_old and lead_old[0] != d) or not lead_new:
            raise MissingShardPatch(f"reshape {tuple(old)} -> {tuple(new)} splits the sharded dim {d} unevenly")
        tgt = lead_new[0]
        inner_old = math.prod(old[k] for k in oi if k > d)
        inner_new = math.prod(new[k] for k in nj if k > tgt)
        per_rank = [s * inner_old for s in spec.sharding_sizes[md]]
        if any(v % inner_new for v in per_rank):
            raise MissingShardPatch("reshape does not keep whole rows of the sharded dim on each rank")
        sizes[md] = tuple(v // inner_new for v in per_rank)
        from ..spec import mesh_coordinate

        local_new[tgt] = sizes[md][mesh_coordinate(spec.mesh, md)]
        placements[md] = Shard(tgt)
    with NO_TF():
        out = local(x).reshape(local_new)
    return wrap(out, spec.mesh, placements, sizes)


@register(torch.Tensor.flatten, torch.flatten)
def _flatten(func, types, args, kwargs):
    x = args[0]
    start = norm_dim(kwargs.get("start_dim", args[1] if len(args) > 1 else 0), x.dim())
    end = norm_dim(kwargs.get("end_dim", args[2] if len(args) > 2 else -1), x.dim())
    shape = list(x.shape)
    new = shape[:start] + [math.prod(shape[start:end + 1])] + shape[end + 1:]
    return x.reshape(new)


@register(torch.Tensor.unflatten, torch.unflatten)
def _unflatten(func, types, args, kwargs):
    x = args[0]
    d = norm_dim(kwargs.get("dim", args[1] if len(args) > 1 else None), x.dim())
    sz = list(kwargs.get("sizes", args[2] if len(args) > 2 else None))
    shape = list(x.shape)
    if -1 in sz:
        sz[sz.index(-1)] = shape[d] // math.prod(s for s in sz if s != -1)
    return x.reshape(shape[:d] + sz + shape[d + 1:])


def _remap(x: ShardTensor, out, perm_new_of_old):
    """Wrap ``out`` whose dim ``perm_new_of_old[d]`` is the old dim ``d`` (None = dropped)."""
    spec = x._spec
    placements = []
    sizes = {}
    for md, p in enumerate(spec.placements):
        if isinstance(p, Shard):
            nd = perm_new_of_old[p.dim]
            if nd is None:
                raise MissingShardPatch("operation removes the sharded dimension")
            placements.append(Shard(nd))
            sizes[md] = spec.sharding_sizes[md]
        else:
            placements.append(p)
    return wrap(out, spec.mesh, placements, sizes)


@register(torch.Tensor.permute, torch.permute)
def _permute(func, types, args, kwargs):
    x = args[0]
    dims = kwargs.get("dims", args[1:] if len(args) > 2 or not isinstance(args[1], (list, tuple)) else args[1])
    dims = [norm_dim(d, x.dim()) for d in dims]
    with NO_TF():
        out = local(x).permute(*dims)
    inv = {old: new for new, old in enumerate(dims)}
    return _remap(x, out, inv)


@register(torch.Tensor.transpose, torch.transpose, torch.Tensor.swapaxes, torch.swapaxes)
def _transpose(func, types, args, kwargs):
    x = args[0]
    a, b = norm_dim(args[1], x.dim()), norm_dim(args[2], x.dim())
    dims = list(range(x.dim()))
    dims[a], dims[b] = dims[b], dims[a]
    return x.permute(*dims)


@register(torch.Tensor.t)
def _t(func, types, args, kwargs):
    return args[0].transpose(0, 1)


@register(torch.Tensor.unsqueeze, torch.unsqueeze)
def _unsqueeze(func, types, args, kwargs):
    x = args[0]
    d = kwargs.get("dim", args[1] if len(args) > 1 else None)
    d = d + x.dim() + 1 if d < 0 else d
    with NO_TF():
        out = local(x).unsqueeze(d)
    return _remap(x, out, {k: (k if k < d else k + 1) for k in range(x.dim())})


@register(torch.Tensor.squeeze, torch.squeeze)
def _squeeze(func, types, args, kwargs):
    x = args[0]
    d = kwargs.get("dim", args[1] if len(args) > 1 else None)
    shape = list(x.shape)
    drop = [k for k in range(x.dim()) if shape[k] == 1] if d is None else \
        [norm_dim(k, x.dim()) for k in (d if isinstance(d, (list, tuple)) else [d]) if shape[norm_dim(k, x.dim())] == 1]
    sharded = x._spec.sharded_tensor_dims()
    drop = [k for k in drop if k not in sharded]
    with NO_TF():
        out = local(x)
        for k in sorted(drop, reverse=True):
            out = out.squeeze(k)
    mapping, n = {}, 0
    for k in range(x.dim()):
        if k in drop:
            mapping[k] = None
        else:
            mapping[k] = n
            n += 1
    return _remap(x, out, mapping)


@register(torch.Tensor.expand, torch.Tensor.expand_as, torch.Tensor.repeat, torch.broadcast_to)
def _expand(func, types, args, kwargs):
    x = args[0]
    if func is torch.Tensor.expand_as:
        target = list(args[1].shape)
    else:
        target = _shape_arg(args, kwargs)
    lead = len(target) - x.dim()
    spec = x._spec
    loc = list(target)
    from ..spec import mesh_coordinate

    for md, p in enumerate(spec.placements):
        if isinstance(p, Shard):
            k = p.dim + lead
            if func is torch.Tensor.repeat:
                if target[k] != 1:
                    raise MissingShardPatch("repeat along a sharded dimension")
            else:
                loc[k] = -1 if target[k] in (-1, x.shape[p.dim]) else None
                if loc[k] is None:
                    raise MissingShardPatch("expand along a sharded dimension")
    with NO_TF():
        out = local(x).repeat(*loc) if func is torch.Tensor.repeat else local(x).expand(*loc)
    return _remap(x, out, {k: k + lead for k in range(x.dim())})


@register(torch.Tensor.__getitem__)
def _getitem(func, types, args, kwargs):
    x, idx = args[0], args[1]
    if not is_st(x):
        raise MissingShardPatch("indexing a plain tensor with a ShardTensor")
    if not isinstance(idx, tuple):
        idx = (idx,)
    if any(isinstance(i, torch.Tensor) for i in idx):
        sharded = x._spec.sharded_tensor_dims()
        pos = [k for k, i in enumerate(idx) if isinstance(i, torch.Tensor)]
        if any(k in sharded for k in pos) or Ellipsis in idx:
            raise MissingShardPatch("advanced indexing on a sharded dimension")
    # expand the ellipsis
    n_real = sum(1 for i in idx if i is not None and i is not Ellipsis)
    full: List = []
    for i in idx:
        if i is Ellipsis:
            full += [slice(None)] * (x.dim() - n_real)
        else:
            full.append(i)
    full += [slice(None)] * (x.dim() - sum(1 for i in full if i is not None))
    sharded = x._spec.sharded_tensor_dims()
    mapping, old, new = {}, 0, 0
    for i in full:
        if i is None:
            new += 1
            continue
        if old in sharded and not (isinstance(i, slice) and i == slice(None)):
            raise MissingShardPatch("slicing / selecting along a sharded dimension needs redistribute()")
        if isinstance(i, int):
            mapping[old] = None
        else:
            mapping[old] = new
            new += 1
        old += 1
    with NO_TF():
        out = local(x)[tuple(local(i) if is_st(i) else i for i in full)]
    return _remap(x, out, mapping)


@register(torch.Tensor.select, torch.select)
def _select(func, types, args, kwargs):
    x = args[0]
    d = norm_dim(kwargs.get("dim", args[1] if len(args) > 1 else None), x.dim())
    i = kwargs.get("index", args[2] if len(args) > 2 else None)
    idx = [slice(None)] * x.dim()
    idx[d] = i
    return x[tuple(idx)]


@register(torch.Tensor.unbind, torch.unbind)
def _unbind(func, types, args, kwargs):
    x = args[0]
    d = norm_dim(kwargs.get("dim", args[1] if len(args) > 1 else 0), x.dim())
    return tuple(x.select(d, i) for i in range(x.shape[d]))


@register(torch.Tensor.chunk, torch.chunk, torch.Tensor.split, torch.split, torch.Tensor.tensor_split)
def _split(func, types, args, kwargs):
    x = args[0]
    d = norm_dim(kwargs.get("dim", args[2] if len(args) > 2 else 0), x.dim())
    if d in x._spec.sharded_tensor_dims():
        raise MissingShardPatch("split / chunk along a sharded dimension")
    with NO_TF():
        pieces = func(local(x), *args[1:], **kwargs)
    return tuple(_remap(x, p, {k: k for k in range(x.dim())}) for p in pieces)


@register(torch.cat, torch.concat, torch.concatenate, torch.stack)
def _cat(func, types, args, kwargs):
    tensors = list(args[0])
    d = kwargs.get("dim", args[1] if len(args) > 1 else 0)
    ref = next(t for t in tensors if is_st(t))
    nd = ref.dim() + (1 if func is torch.stack else 0)
    d = norm_dim(d, nd)
    if func is not torch.stack and d in ref._spec.sharded_tensor_dims():
        raise MissingShardPatch("concatenation along a sharded dimension")
    for t in tensors:
        if is_st(t) and not t._spec.same_layout(ref._spec):
            raise MissingShardPatch("concatenating ShardTensors with different layouts")
    from ..grad_ops import reduce_grad_over_mesh

    locs = [local(t) if is_st(t) else reduce_grad_over_mesh(t, ref._spec.mesh) for t in tensors]
    with NO_TF():
        out = func(locs, dim=d)
    if func is torch.stack:
        return _remap(ref, out, {k: (k if k < d else k + 1) for k in range(ref.dim())})
    return _remap(ref, out, {k: k for k in range(ref.dim())})
