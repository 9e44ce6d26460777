"""Reductions and contractions over sharded dimensions.

Parity: ``physicsnemo/domain_parallel/custom_ops/_reductions.py`` (``ShardedSum`` /
``ShardedMean``: local reduction, result ``Partial("sum")`` when a sharded dim is reduced; the
mean weights the local mean by ``local / global`` extent) and the Partial results of
contractions over the sharded token dimension that Transolver relies on
(``nn/module/physics_attention.py:120-206``).  ``max`` / ``min`` / ``amax`` / ``amin`` over a
sharded dim reduce locally and finish with a MAX / MIN all-reduce.
"""
from __future__ import annotations

import math
import re

import torch
import torch.distributed as dist
from torch.distributed.tensor import Partial, Replicate, Shard

from ..grad_ops import reduce_grad_over_mesh
from ._common import MissingShardPatch, NO_TF, ShardTensor, is_st, local, norm_dim, param, register, resolved, wrap


def _dims(x, args, kwargs):
    d = kwargs.get("dim", kwargs.get("axis", args[1] if len(args) > 1 and not isinstance(args[1], torch.dtype) else None))
    if d is None or (isinstance(d, (list, tuple)) and len(d) == 0):
        return list(range(x.dim()))
    d = [d] if isinstance(d, int) else list(d)
    return [norm_dim(k, x.dim()) for k in d]


def _reduce(func_name, x: ShardTensor, dims, keepdim, dtype=None):
    x = resolved(x)
    spec = x._spec
    loc = local(x)
    sharded = {p.dim: md for md, p in enumerate(spec.placements) if isinstance(p, Shard)}
    hit = [d for d in dims if d in sharded]
    with NO_TF():
        kw = {"dtype": dtype} if dtype is not None else {}
        out = loc.sum(dim=dims, keepdim=keepdim, **kw)
        if func_name == "mean":
            count = math.prod(x.shape[d] for d in dims)
            out = out / count
    placements, sizes = [], {}
    removed = sorted(dims)
    for md, p in enumerate(spec.placements):
        if isinstance(p, Shard):
            if p.dim in hit:
                placements.append(Partial("sum"))
            else:
                nd = p.dim if keepdim else p.dim - sum(1 for r in removed if r < p.dim)
                placements.append(Shard(nd))
                sizes[md] = spec.sharding_sizes[md]
        else:
            placements.append(p)
    return wrap(out, spec.mesh, placements, sizes)


@register(torch.sum, torch.Tensor.sum, torch.mean, torch.Tensor.mean)
def _sum_mean(func, types, args, kwargs):
    x = args[0]
    name = "mean" if func in (torch.mean, torch.Tensor.mean) else "sum"
    return _reduce(name, x, _dims(x, args, kwargs), kwargs.get("keepdim", False), kwargs.get("dtype"))


class _AllReduceMinMax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, v, group, is_max):
        out = v.contiguous().clone()
        dist.all_reduce(out, op=dist.ReduceOp.MAX if is_max else dist.ReduceOp.MIN, group=group)
        ctx.save_for_backward(v, out)
        return out

    @staticmethod
    def backward(ctx, g):
        v, out = ctx.saved_tensors
        return g * (v == out).to(g.dtype), None, None


@register(torch.amax, torch.Tensor.amax, torch.amin, torch.Tensor.amin)
def _amax(func, types, args, kwargs):
    x = resolved(args[0])
    dims = _dims(x, args, kwargs)
    keepdim = kwargs.get("keepdim", False)
    is_max = func in (torch.amax, torch.Tensor.amax)
    spec = x._spec
    with NO_TF():
        out = local(x).amax(dim=dims, keepdim=keepdim) if is_max else local(x).amin(dim=dims, keepdim=keepdim)
    placements, sizes = [], {}
    removed = sorted(dims)
    for md, p in enumerate(spec.placements):
        if isinstance(p, Shard) and p.dim in dims:
            out = _AllReduceMinMax.apply(out, spec.mesh.get_group(md), is_max)
            placements.append(Replicate())
        elif isinstance(p, Shard):
            nd = p.dim if keepdim else p.dim - sum(1 for r in removed if r < p.dim)
            placements.append(Shard(nd))
            sizes[md] = spec.sharding_sizes[md]
        else:
            placements.append(p)
    return wrap(out, spec.mesh, placements, sizes)


@register(torch.nn.functional.mse_loss, torch.nn.functional.l1_loss, torch.nn.functional.smooth_l1_loss,
          torch.nn.functional.huber_loss)
def _elementwise_loss(func, types, args, kwargs):
    inp, tgt = args[0], args[1]
    reduction = kwargs.get("reduction", "mean")
    kw = {k: v for k, v in kwargs.items() if k != "reduction"}
    ref = inp if is_st(inp) else tgt
    if is_st(inp) and is_st(tgt) and not inp._spec.same_layout(tgt._spec):
        tgt = tgt.redistribute(placements=inp._spec.placements)
    li = local(resolved(inp)) if is_st(inp) else reduce_grad_over_mesh(inp, ref._spec.mesh)
    lt = local(resolved(tgt)) if is_st(tgt) else tgt
    with NO_TF():
        per = func(li, lt, reduction="none", **kw)
    out = ShardTensor(per, resolved(ref)._spec.with_(dtype=per.dtype))
    if reduction == "none":
        return out
    return out.mean() if reduction == "mean" else out.sum()


@register(torch.matmul, torch.Tensor.matmul, torch.Tensor.__matmul__, torch.bmm, torch.Tensor.bmm)
def _matmul(func, types, args, kwargs):
    a, b = args[0], args[1]
    if is_st(a) and is_st(b):
        a, b = resolved(a), resolved(b)
        sa = {p.dim: md for md, p in enumerate(a._spec.placements) if isinstance(p, Shard)}
        sb = {p.dim: md for md, p in enumerate(b._spec.placements) if isinstance(p, Shard)}
        ka, kb = a.dim() - 1, b.dim() - 2
        if ka in sa and kb in sb and sa[ka] == sb[kb] and a._spec.sharding_sizes[sa[ka]] == b._spec.sharding_sizes[sb[kb]]:
            # contraction over the sharded dimension: local product, result is a partial sum
            with NO_TF():
                out = torch.matmul(local(a), local(b))
            placements = [Partial("sum") if md == sa[ka] else p for md, p in enumerate(a._spec.placements)]
            if any(isinstance(p, Shard) for p in placements):
                raise MissingShardPatch("matmul with additional sharded batch dims")
            return wrap(out, a._spec.mesh, placements, {})
    from ..local_rule import apply_local_rule

    return apply_local_rule(func, args, kwargs)


@register(torch.einsum)
def _einsum(func, types, args, kwargs):
    eq = args[0]
    ops = list(args[1]) if len(args) == 2 and isinstance(args[1], (list, tuple)) else list(args[1:])
    sts = [o for o in ops if is_st(o)]
    mesh = sts[0]._spec.mesh
    lhs, rhs = eq.replace(" ", "").split("->")
    terms = lhs.split(",")
    ops = [resolved(o) if is_st(o) else o for o in ops]
    letters = {}  # letter -> (mesh_dim, sizes)
    for term, o in zip(terms, ops):
        if is_st(o):
            for md, p in enumerate(o._spec.placements):
                if isinstance(p, Shard):
                    letters.setdefault(term[p.dim], (md, o._spec.sharding_sizes[md]))
    # every operand carrying a sharded letter must be sharded on it
    for term, o in zip(terms, ops):
        for ch, (md, sizes) in letters.items():
            if ch in term:
                if not is_st(o) or o._spec.shard_dim_of(md) != term.index(ch):
                    raise MissingShardPatch(f"einsum '{eq}': operand is not sharded on index '{ch}' like its partner")
    locs = [local(o) if is_st(o) else reduce_grad_over_mesh(o, mesh) for o in ops]
    with NO_TF():
        out = torch.einsum(eq, *locs)
    placements = [Replicate()] * mesh.ndim
    sizes = {}
    for ch, (md, sz) in letters.items():
        if ch in rhs:
            placements[md] = Shard(rhs.index(ch))
            sizes[md] = sz
        else:
            placements[md] = Partial("sum")
    return wrap(out, mesh, placements, sizes)
