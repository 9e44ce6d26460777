"""Padding, pooling and resampling on spatially sharded inputs.

Parity: ``physicsnemo/domain_parallel/shard_utils/padding.py`` (only edge ranks pad; circular
padding becomes a periodic halo), ``pooling_patches.py`` (``stride == kernel`` and divisible shard
sizes: no halo), ``unpooling_patches.py`` (``F.interpolate``: nearest with integer scale factors is
local; linear modes use a one-row halo and crop).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch.distributed.tensor import Shard

from .. import collectives as C
from ._common import MissingShardPatch, NO_TF, ShardTensor, is_st, local, norm_dim, register, resolved, wrap


@register(F.pad)
def _pad(func, types, args, kwargs):
    x = resolved(args[0])
    pad = list(kwargs.get("pad", args[1] if len(args) > 1 else None))
    mode = kwargs.get("mode", args[2] if len(args) > 2 else "constant")
    value = kwargs.get("value", args[3] if len(args) > 3 else None)
    spec = x._spec
    nd = x.dim()
    sharded = {p.dim: md for md, p in enumerate(spec.placements) if isinstance(p, Shard)}
    loc = local(x)
    sizes = {md: list(s) for md, s in spec.sharding_sizes.items()}
    local_pad = list(pad)
    for j in range(len(pad) // 2):
        d = nd - 1 - j
        lo, hi = pad[2 * j], pad[2 * j + 1]
        if d not in sharded or (lo == 0 and hi == 0):
            continue
        md = sharded[d]
        n, r = spec.mesh.size(md), spec.mesh.get_local_rank(md)
        if mode == "circular":
            if lo != hi:
                raise MissingShardPatch("asymmetric circular padding on a sharded dimension")
            with NO_TF():
                loc = C.HaloPadding.apply(loc, d, lo, 0, spec.mesh.get_group(md), tuple(sizes[md]), True)
            # interior ranks received rows they must not keep
            keep_lo = lo if r == 0 else 0
            keep_hi = hi if r == n - 1 else 0
            with NO_TF():
                loc = loc.narrow(d, lo - keep_lo, loc.shape[d] - (lo - keep_lo) - (hi - keep_hi))
            local_pad[2 * j] = local_pad[2 * j + 1] = 0
        elif mode in ("constant", "replicate", "reflect"):
            if mode == "reflect" and n > 1 and (lo >= sizes[md][0] or hi >= sizes[md][-1]):
                raise MissingShardPatch("reflect padding wider than the edge shard")
            local_pad[2 * j] = lo if r == 0 else 0
            local_pad[2 * j + 1] = hi if r == n - 1 else 0
        else:
            raise MissingShardPatch(f"padding mode {mode} on a sharded dimension")
        sizes[md][0] += lo
        sizes[md][-1] += hi
    with NO_TF():
        if any(local_pad):
            out = F.pad(loc, local_pad, mode=mode if mode != "circular" else "constant", value=value)
        else:
            out = loc
    return wrap(out, spec.mesh, spec.placements, {md: tuple(s) for md, s in sizes.items()})


def _pool(func, types, args, kwargs):
    x = resolved(args[0])
    spec = x._spec
    nsp = x.dim() - 2
    k = kwargs.get("kernel_size", args[1] if len(args) > 1 else None)
    s = kwargs.get("stride", args[2] if len(args) > 2 else None) or k
    pad = kwargs.get("padding", args[3] if len(args) > 3 else 0)
    tup = lambda v: tuple(v) if isinstance(v, (list, tuple)) else (v,) * nsp  # noqa: E731
    k, s, pad = tup(k), tup(s), tup(pad)
    sizes = dict(spec.sharding_sizes)
    for md, p in enumerate(spec.placements):
        if isinstance(p, Shard) and p.dim >= 2:
            i = p.dim - 2
            if k[i] != s[i] or pad[i] != 0:
                raise MissingShardPatch("pooling on a sharded dimension needs stride == kernel and no padding")
            if any(v % k[i] for v in spec.sharding_sizes[md]):
                raise MissingShardPatch("pooling needs shard sizes divisible by the kernel")
            sizes[md] = tuple(v // k[i] for v in spec.sharding_sizes[md])
    with NO_TF():
        out = func(local(x), *args[1:], **kwargs)
    if isinstance(out, tuple):
        return tuple(wrap(o, spec.mesh, spec.placements, sizes) for o in out)
    return wrap(out, spec.mesh, spec.placements, sizes)


for _f in (F.avg_pool1d, F.avg_pool2d, F.avg_pool3d, F.max_pool1d, F.max_pool2d, F.max_pool3d):
    ShardTensor.register_function_handler(_f, _pool)


@register(F.interpolate)
def _interpolate(func, types, args, kwargs):
    names = ["input", "size", "scale_factor", "mode", "align_corners", "recompute_scale_factor", "antialias"]
    a = dict(zip(names, args))
    a.update(kwargs)
    x = resolved(a["input"])
    spec = x._spec
    nsp = x.dim() - 2
    mode = a.get("mode", "nearest")
    sf = a.get("scale_factor")
    size = a.get("size")
    if sf is None:
        if size is None:
            raise ValueError("either size or scale_factor is required")
        size = tuple(size) if isinstance(size, (list, tuple)) else (size,) * nsp
        sf = tuple(size[i] / x.shape[2 + i] for i in range(nsp))
    sf = tuple(sf) if isinstance(sf, (list, tuple)) else (sf,) * nsp
    sharded = {p.dim: md for md, p in enumerate(spec.placements) if isinstance(p, Shard) and p.dim >= 2}
    for d in sharded:
        if float(sf[d - 2]) != int(sf[d - 2]) or sf[d - 2] < 1:
            raise MissingShardPatch("interpolation along a sharded dimension needs an integer up-scaling factor")
    sizes = dict(spec.sharding_sizes)
    loc = local(x)
    if mode in ("nearest", "nearest-exact") or not sharded:
        with NO_TF():
            out = F.interpolate(loc, scale_factor=[float(s) for s in sf], mode=mode,
                                **({"align_corners": a["align_corners"]} if a.get("align_corners") is not None else {}))
        for d, md in sharded.items():
            sizes[md] = tuple(int(v * sf[d - 2]) for v in spec.sharding_sizes[md])
        return wrap(out, spec.mesh, spec.placements, sizes)
    if a.get("align_corners"):
        raise MissingShardPatch("align_corners=True interpolation on a sharded dimension")
    # linear family: one row of halo, replicate-extended at the domain edges, then crop
    crops = {}
    for d, md in sharded.items():
        n, r = spec.mesh.size(md), spec.mesh.get_local_rank(md)
        with NO_TF():
            loc = C.HaloPadding.apply(loc, d, 1, 0, spec.mesh.get_group(md), spec.sharding_sizes[md], False)
            idx = [slice(None)] * loc.dim()
            if r == 0:
                idx[d] = slice(0, 1)
                loc = torch.cat([loc[tuple(idx)], loc], dim=d)
            if r == n - 1:
                idx[d] = slice(loc.shape[d] - 1, loc.shape[d])
                loc = torch.cat([loc, loc[tuple(idx)]], dim=d)
        f = int(sf[d - 2])
        crops[d] = (f, f)
        sizes[md] = tuple(v * f for v in spec.sharding_sizes[md])
    with NO_TF():
        out = F.interpolate(loc, scale_factor=[float(s) for s in sf], mode=mode, align_corners=False)
        for d, (lo, hi) in crops.items():
            out = out.narrow(d, lo, out.shape[d] - lo - hi)
    return wrap(out, spec.mesh, spec.placements, sizes)
