"""Convolutions on spatially sharded inputs: halo exchange + local convolution.

Parity: ``physicsnemo/domain_parallel/shard_utils/conv_patches.py`` — halo per sharded spatial
dim = ``dilation * (kernel - 1) // 2`` for odd kernels with stride 1; even kernels with
``stride == kernel`` and no padding need no halo (``:72-135``); the convolution's own padding on
a sharded dim becomes zero padding of the domain edges only (``:192-287``); output shard sizes
are computed analytically for every rank (``:291-401``); transposed convolutions only in the
``stride == kernel`` case.  Strided odd kernels are supported when every shard start is a
multiple of the stride.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F
from torch.distributed.tensor import Shard

from .. import collectives as C
from ._common import MissingShardPatch, NO_TF, ShardTensor, is_st, local, param, register, resolved, wrap


def _tup(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


def _bf16_mode(t: torch.Tensor) -> bool:
    if t.dtype == torch.bfloat16:
        return True
    return t.is_cuda and torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16


def _fused_halo_conv(loc, w, b, spec, stride, padding, dilation, groups):
    """The halo-fused tcgen05 path (``parallel/halo_conv.py``) when it covers this call, else ``None``.

    Conditions: CUDA + NCCL, bf16 compute, 2-D 3×3 / stride 1 / padding 1 / no dilation / one group, input sharded on
    the height only (tensor dim 2) over a 1-D mesh dimension, every shard a multiple of 8 rows.
    """
    if loc.dim() != 4 or not loc.is_cuda or not _bf16_mode(loc) or groups != 1:
        return None
    if tuple(w.shape[2:]) != (3, 3) or stride != (1, 1) or dilation != (1, 1) or tuple(padding) != (1, 1):
        return None
    shards = [(md, p) for md, p in enumerate(spec.placements) if isinstance(p, Shard)]
    if len(shards) != 1 or shards[0][1].dim != 2:
        return None
    md = shards[0][0]
    sizes = spec.sharding_sizes[md]
    if any(v % 8 or v == 0 for v in sizes):
        return None
    from ..halo_conv import get_halo_runtime, halo_conv2d_3x3, halo_conv_supported
    from ..peer import peer_available

    if not peer_available(loc):
        return None
    rt = get_halo_runtime(spec.mesh.get_group(md))
    if not halo_conv_supported(loc, w, rt):
        return None
    with NO_TF():
        return halo_conv2d_3x3(loc, w, b, rt)


def _conv(func, types, args, kwargs):
    names = ["input", "weight", "bias", "stride", "padding", "dilation", "groups"]
    a = dict(zip(names, args))
    a.update(kwargs)
    x = a["input"]
    if not is_st(x):
        raise MissingShardPatch("convolution with sharded weights but a plain input")
    x = resolved(x)
    spec = x._spec
    nsp = x.dim() - 2
    w = param(a["weight"], spec.mesh)
    b = param(a.get("bias"), spec.mesh)
    stride = _tup(a.get("stride", 1), nsp)
    dilation = _tup(a.get("dilation", 1), nsp)
    groups = a.get("groups", 1)
    padding = a.get("padding", 0)
    ksize = w.shape[2:]
    if isinstance(padding, str):
        if padding == "valid":
            padding = (0,) * nsp
        elif padding == "same":
            if any(s != 1 for s in stride):
                raise MissingShardPatch("padding='same' needs stride 1")
            if any((dilation[i] * (ksize[i] - 1)) % 2 for i in range(nsp)):
                raise MissingShardPatch("padding='same' with an even receptive field on a sharded input")
            padding = tuple(dilation[i] * (ksize[i] - 1) // 2 for i in range(nsp))
    padding = list(_tup(padding, nsp))
    loc = local(x)
    placements = list(spec.placements)
    if nsp == 2 and not isinstance(padding, str):
        fused = _fused_halo_conv(loc, w, b, spec, stride, _tup(padding, nsp), dilation, groups)
        if fused is not None:
            return wrap(fused, spec.mesh, placements, dict(spec.sharding_sizes))
    sizes = {}
    for md, p in enumerate(spec.placements):
        if not isinstance(p, Shard):
            continue
        if p.dim < 2:
            if p.dim == 1:
                raise MissingShardPatch("convolution over a channel-sharded input")
            sizes[md] = spec.sharding_sizes[md]
            continue
        i = p.dim - 2
        k, s, d, pad = ksize[i], stride[i], dilation[i], padding[i]
        in_sizes = spec.sharding_sizes[md]
        group = spec.mesh.get_group(md)
        rf = d * (k - 1) + 1
        if s == k and d == 1 and pad == 0:
            if any(v % s for v in in_sizes):
                raise MissingShardPatch("stride == kernel convolution needs shard sizes divisible by the stride")
            sizes[md] = tuple(v // s for v in in_sizes)
            continue
        if rf % 2 == 0:
            raise MissingShardPatch(f"even receptive field {rf} with stride {s} on a sharded dimension")
        halo = rf // 2
        if pad > halo:
            raise MissingShardPatch("padding larger than the halo on a sharded dimension")
        n = len(in_sizes)
        starts = [sum(in_sizes[:r]) for r in range(n)]
        if s > 1 and (pad != halo or any(st % s for st in starts)):
            raise MissingShardPatch(
                "strided convolution on a sharded dimension needs padding == kernel // 2 and every shard "
                "starting on a multiple of the stride")
        # local tensor = [halo rows of the left neighbour | shard | halo rows of the right neighbour], with
        # `pad` zero rows instead at the two ends of the domain; an unpadded local convolution then yields
        # exactly the outputs whose window centre lies in this shard.
        loc = C.HaloPadding.apply(loc, p.dim, halo, pad, group, in_sizes, False)
        if s == 1:
            sizes[md] = tuple(v - (halo - pad) * (int(r == 0) + int(r == n - 1)) for r, v in enumerate(in_sizes))
        else:
            sizes[md] = tuple(-(-v // s) for v in in_sizes)
        padding[i] = 0
    with NO_TF():
        from ...ops import conv as _oc

        if (nsp == 2 and loc.is_cuda and _bf16_mode(loc) and all(pd == ksize[i] // 2 for i, pd in enumerate(padding))
                and _oc.supported(loc, w, stride, tuple(padding), dilation, groups)):
            out = _oc.conv2d_same(loc, w, b)        # no halo left to fetch (1×1, or the padded copy already holds it)
        else:
            out = func(loc, w, b, stride, tuple(padding), dilation, groups)
    for md, p in enumerate(spec.placements):
        if isinstance(p, Shard) and p.dim >= 2:
            want = sizes[md][spec.mesh.get_local_rank(md)]
            got = out.shape[p.dim]
            if got != want:
                raise MissingShardPatch(
                    f"sharded convolution produced {got} rows on this rank where {want} were expected "
                    f"(kernel {tuple(ksize)}, stride {stride}, padding {a.get('padding', 0)})")
    return wrap(out, spec.mesh, placements, sizes)


for _f in (F.conv1d, F.conv2d, F.conv3d):
    ShardTensor.register_function_handler(_f, _conv)


def _conv_transpose(func, types, args, kwargs):
    names = ["input", "weight", "bias", "stride", "padding", "output_padding", "groups", "dilation"]
    a = dict(zip(names, args))
    a.update(kwargs)
    x = resolved(a["input"])
    spec = x._spec
    nsp = x.dim() - 2
    w = param(a["weight"], spec.mesh)
    b = param(a.get("bias"), spec.mesh)
    stride = _tup(a.get("stride", 1), nsp)
    padding = _tup(a.get("padding", 0), nsp)
    opad = _tup(a.get("output_padding", 0), nsp)
    dilation = _tup(a.get("dilation", 1), nsp)
    sizes = {}
    for md, p in enumerate(spec.placements):
        if isinstance(p, Shard) and p.dim >= 2:
            i = p.dim - 2
            if not (stride[i] == w.shape[2 + i] and padding[i] == 0 and opad[i] == 0 and dilation[i] == 1):
                raise MissingShardPatch("transposed convolution on a sharded dim needs stride == kernel, no padding")
            sizes[md] = tuple(v * stride[i] for v in spec.sharding_sizes[md])
        elif isinstance(p, Shard):
            sizes[md] = spec.sharding_sizes[md]
    with NO_TF():
        out = func(local(x), w, b, stride, padding, opad, a.get("groups", 1), dilation)
    return wrap(out, spec.mesh, spec.placements, sizes)


for _f in (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d):
    ShardTensor.register_function_handler(_f, _conv_transpose)
