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


def _fused_sharded_gn(x: ShardTensor, G: int, w, b, eps: float, silu: bool):
    """GroupNorm(+SiLU) on the peer-memory kernels when they cover this tensor, else ``None``.

    Conditions: CUDA + NCCL, 4-D bf16 / fp32 input sharded on one spatial dim over a 1-D mesh dimension, affine
    parameters present.  The statistics cross the ranks inside the normalising kernel (``ops/group_norm.py``).
    """
    spec = x._spec
    loc = local(x)
    if w is None or b is None or loc.dim() != 4 or not loc.is_cuda:
        return None
    shards = [(md, p) for md, p in enumerate(spec.placements) if isinstance(p, Shard)]
    if len(shards) != 1 or shards[0][1].dim < 2:
        return None
    from ...ops import group_norm as _gn
    from ..peer import get_runtime, peer_available

    if not peer_available(loc):
        return None
    md = shards[0][0]
    rt = get_runtime(spec.mesh.get_group(md), "compute")
    if loc.dtype not in (torch.bfloat16, torch.float32) or not _gn.sharded_supported(loc, G, rt):
        return None
    with NO_TF():
        out = _gn.group_norm_sharded(loc, G, w, b, eps, silu, rt, math.prod(x.shape[2:]))
    return wrap(out, spec.mesh, spec.placements, spec.sharding_sizes)


def group_norm_act(x: ShardTensor, num_groups: int, weight, bias, eps: float, act: str | None):
    """``act(group_norm(x))`` for a ShardTensor: one fused kernel pair when ``act`` is SiLU (or absent), else the
    composition.  Entry point of ``nn.GroupNorm`` for sharded inputs."""
    x = resolved(x)
    if act in (None, "silu"):
        w, b = param(weight, x._spec.mesh), param(bias, x._spec.mesh)
        out = _fused_sharded_gn(x, num_groups, w, b, eps, act == "silu")
        if out is not None:
            return out
    y = F.group_norm(x, num_groups, weight, bias, eps)
    if act is None:
        return y
    return getattr(F, act)(y) if hasattr(F, act) else getattr(torch, act)(y)


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
    fused = _fused_sharded_gn(x, G, w, b, eps, False)
    if fused is not None:
        return fused
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
