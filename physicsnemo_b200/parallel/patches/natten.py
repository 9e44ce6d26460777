"""Neighbourhood attention on spatially sharded token grids.

Parity: ``physicsnemo/domain_parallel/shard_utils/natten_patches.py:141-277``.  Every query attends to a
``kernel_size`` window of keys around it (windows that would leave the grid are shifted inwards).  On a shard, the keys
and values of ``(kernel_size // 2) · dilation`` rows of each neighbour are needed: q, k and v receive that halo
(differentiable exchange), the single-device operator runs on the padded shard, and the halo rows of the RESULT are
dropped.  Interior shards then see complete windows; a shard at the border of the grid has no halo on the outer side
and shifts its windows inwards exactly as the global operator does.  Dilated windows stay aligned only if every shard
starts at a multiple of the dilation, which is checked.
"""
from __future__ import annotations

from torch.distributed.tensor import Shard

from ...nn.functional import natten as _na
from .. import collectives as C
from ._common import MissingShardPatch, NO_TF, ShardTensor, is_st, local, register, resolved, wrap


def _as_tuple(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


def _make_rule(nd: int):
    def rule(func, types, args, kwargs):
        q, k, v = args[0], args[1], args[2]
        kernel_size = kwargs.get("kernel_size", args[3] if len(args) > 3 else None)
        dilation = kwargs.get("dilation", args[4] if len(args) > 4 else 1)
        rest = {key: val for key, val in kwargs.items() if key not in ("kernel_size", "dilation")}
        if not all(is_st(t) for t in (q, k, v)):
            raise MissingShardPatch("neighbourhood attention needs q, k and v sharded alike")
        q, k, v = resolved(q), resolved(k), resolved(v)
        spec = q._spec
        if k._spec.placements != spec.placements or v._spec.placements != spec.placements:
            raise MissingShardPatch("q, k and v must share one sharding")
        kern, dil = _as_tuple(kernel_size, nd), _as_tuple(dilation, nd)
        lq, lk, lv = local(q), local(k), local(v)
        crops = []
        for md, p in enumerate(spec.placements):
            if not isinstance(p, Shard):
                continue
            d = p.dim
            if not 1 <= d <= nd:
                raise MissingShardPatch("only the spatial dimensions of a token grid may be sharded")
            sizes = [int(s) for s in spec.sharding_sizes[md]]
            halo = (kern[d - 1] // 2) * dil[d - 1]
            if halo == 0:
                continue
            starts = [sum(sizes[:i]) for i in range(len(sizes))]
            if dil[d - 1] > 1 and any(s % dil[d - 1] for s in starts):
                raise MissingShardPatch("with dilation every shard must start at a multiple of the dilation")
            if min(sizes) < halo:
                raise MissingShardPatch("a shard is narrower than the attention halo")
            group, r, n = spec.mesh.get_group(md), spec.mesh.get_local_rank(md), spec.mesh.size(md)
            with NO_TF():
                lq, lk, lv = (C.HaloPadding.apply(t, d, halo, 0, group, tuple(sizes), False) for t in (lq, lk, lv))
            crops.append((d, halo if r > 0 else 0, halo if r < n - 1 else 0))
        with NO_TF():
            out = getattr(_na, func.__name__)(lq, lk, lv, kernel_size, dilation=dilation, **rest)
            for d, left, right in crops:                                   # drop the halo rows of the result
                out = out.narrow(d, left, out.shape[d] - left - right)
        return wrap(out, spec.mesh, spec.placements, spec.sharding_sizes)

    return rule


for _nd, _fn in ((1, _na.na1d), (2, _na.na2d), (3, _na.na3d)):
    register(_fn)(_make_rule(_nd))
