"""Normalisations whose statistics span sharded dimensions.

Parity: ``physicsnemo/domain_parallel/shard_utils/normalization_patches.py`` —
``PartialGroupNorm``: local Σx and Σx² per (sample, group), one packed all-reduce, global
mean / rstd with the *global* element count (uneven shards), normalise + affine locally; the
backward packs (Σ dx̂, Σ dx̂·x̂) into one all-reduce.  Here the backward falls out of autograd
through the differentiable all-reduce.  ``layer_norm`` over unsharded trailing dims and
``batch_norm`` in evaluation mode go through the generic local rule.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch.distributed.tensor import Shard

from .. import collectives as C
from ._common import MissingShardPatch, NO_TF, ShardTensor, is_st, local, param, register, resolved, wrap


@register(F.group_norm)
def _group_norm(func, types, args, kwargs):
    names = ["input", "num_groups", "weight", "bias", "eps"]
    a = dict(zip(names, args))
    a.update(kwargs)
    x = resolved(a["input"])
    spec = x._spec
    G = a["num_groups"]
    w, b = param(a.get("weight"), spec.mesh), param(a.get("bias"), spec.mesh)
    eps = a.get("eps", 1e-5)
    sharded = {p.dim: md for md, p in enumerate(spec.placements) if isinstance(p, Shard)}
    if 1 in sharded:
        raise MissingShardPatch("group_norm over a channel-sharded input")
    spatial = [d for d in sharded if d >= 2]
    loc = local(x)
    if not spatial:
        with NO_TF():
            out = F.group_norm(loc, G, w, b, eps)
        return wrap(out, spec.mesh, spec.placements, spec.sharding_sizes)
    N, Cc = loc.shape[0], loc.shape[1]
    with NO_TF():
        acc = torch.float32 if loc.dtype in (torch.bfloat16, torch.float16) else loc.dtype
        xg = loc.reshape(N, G, -1).to(acc)
        stats = torch.stack([xg.sum(-1), (xg * xg).sum(-1)])  # (2, N, G)
        for d in spatial:
            stats = C.AllReduceSum.apply(stats, spec.mesh.get_group(sharded[d]))
        count = (Cc // G) * math.prod(x.shape[2:])  # global number of elements per group
        mean = stats[0] / count
        var = (stats[1] / count - mean * mean).clamp_min(0.0)
        rstd = torch.rsqrt(var + eps)
        y = ((xg - mean.unsqueeze(-1)) * rstd.unsqueeze(-1)).reshape(loc.shape)
        shape = [1, Cc] + [1] * (loc.dim() - 2)
        if w is not None:
            y = y * w.to(acc).reshape(shape)
        if b is not None:
            y = y + b.to(acc).reshape(shape)
        out = y.to(loc.dtype)
    return wrap(out, spec.mesh, spec.placements, spec.sharding_sizes)


@register(F.instance_norm)
def _instance_norm(func, types, args, kwargs):
    x = args[0]
    names = ["input", "running_mean", "running_var", "weight", "bias", "use_input_stats", "momentum", "eps"]
    a = dict(zip(names, args))
    a.update(kwargs)
    if a.get("running_mean") is not None and not a.get("use_input_stats", True):
        from ..local_rule import apply_local_rule

        return apply_local_rule(func, args, kwargs)
    C_ = x.shape[1]
    return F.group_norm(x, C_, a.get("weight"), a.get("bias"), a.get("eps", 1e-5))
