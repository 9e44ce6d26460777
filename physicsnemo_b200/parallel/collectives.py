"""Differentiable collectives on local shards.

Gradient convention of the domain-parallel layer: every rank differentiates the *sum over
ranks* of the per-rank partial losses with respect to its local quantities.  A value that is
replicated and consumed by all ranks therefore receives, on each rank, only that rank's share
of its gradient, and the backward of the collective that produced it sums the shares.

Parity: the reference obtains the same semantics from DTensor placements
(``physicsnemo/domain_parallel/_shard_redistribute.py``, ``shard_utils/halo.py``,
``shard_utils/ring.py``, ``shard_utils/grad_ops.py``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..distributed.utils import _all_to_all


def _world(group) -> int:
    return dist.get_world_size(group=group)


def _global_rank(group, group_rank: int) -> int:
    return dist.get_global_rank(group, group_rank) if group is not None else group_rank


class AllReduceSum(torch.autograd.Function):
    """Sum over the group forward (Partial → Replicate); sum of gradient shares backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.contiguous().clone()
        if _world(group) > 1:
            if y.dtype in (torch.bfloat16, torch.float16):
                z = y.float()
                dist.all_reduce(z, group=group)
                y = z.to(y.dtype)
            else:
                dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        if _world(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g, None


class GradAllReduce(torch.autograd.Function):
    """Identity forward; all-reduce of the gradient backward (replicated parameters used on shards)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        if _world(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g, None


class AllGatherV(torch.autograd.Function):
    """Concatenate uneven shards along ``dim`` (Shard → Replicate); backward keeps the own slice of the summed gradient."""

    @staticmethod
    def forward(ctx, x, sizes, dim, group):
        ctx.sizes, ctx.dim, ctx.group = tuple(sizes), dim, group
        n = _world(group)
        if n == 1:
            return x.clone()
        biggest = max(sizes)
        xs = x.contiguous()
        if xs.shape[dim] < biggest:
            pad_shape = list(xs.shape)
            pad_shape[dim] = biggest - xs.shape[dim]
            xs = torch.cat([xs, xs.new_zeros(pad_shape)], dim=dim)
        outs = [torch.empty_like(xs) for _ in range(n)]
        dist.all_gather(outs, xs.contiguous(), group=group)
        return torch.cat([o.narrow(dim, 0, s) for o, s in zip(outs, sizes)], dim=dim)

    @staticmethod
    def backward(ctx, g):
        n = _world(ctx.group)
        if n == 1:
            return g, None, None, None
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(group=ctx.group)
        start = sum(ctx.sizes[:r])
        return g.narrow(ctx.dim, start, ctx.sizes[r]).contiguous(), None, None, None


class SliceLocal(torch.autograd.Function):
    """Keep this rank's slice of a replicated tensor (Replicate → Shard); backward zero-pads the share."""

    @staticmethod
    def forward(ctx, x, start, length, dim):
        ctx.start, ctx.length, ctx.dim, ctx.full = start, length, dim, x.shape[dim]
        return x.narrow(dim, start, length).contiguous()

    @staticmethod
    def backward(ctx, g):
        shape = list(g.shape)
        shape[ctx.dim] = ctx.full
        out = g.new_zeros(shape)
        out.narrow(ctx.dim, ctx.start, ctx.length).copy_(g)
        return out, None, None, None


def _exchange_with_neighbours(send_left: Optional[torch.Tensor], send_right: Optional[torch.Tensor],
                              recv_left_shape, recv_right_shape, group, like: torch.Tensor, periodic: bool = False):
    """Send slabs to the left / right neighbour of the 1-D group and receive theirs.

    Returns ``(from_left, from_right)``; ``None`` where there is no neighbour.
    """
    n, r = _world(group), dist.get_rank(group=group)
    left = (r - 1) % n if (periodic or r > 0) else None
    right = (r + 1) % n if (periodic or r < n - 1) else None
    ops, from_left, from_right = [], None, None
    if left is not None and recv_left_shape is not None:
        from_left = like.new_empty(recv_left_shape)
        ops.append(dist.P2POp(dist.irecv, from_left, _global_rank(group, left), group=group))
    if right is not None and recv_right_shape is not None:
        from_right = like.new_empty(recv_right_shape)
        ops.append(dist.P2POp(dist.irecv, from_right, _global_rank(group, right), group=group))
    if left is not None and send_left is not None:
        ops.append(dist.P2POp(dist.isend, send_left.contiguous(), _global_rank(group, left), group=group))
    if right is not None and send_right is not None:
        ops.append(dist.P2POp(dist.isend, send_right.contiguous(), _global_rank(group, right), group=group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return from_left, from_right


class HaloPadding(torch.autograd.Function):
    """Pad a shard along ``dim`` with ``halo`` rows of each neighbour (zeros of width
    ``edge_pad`` at the domain edges).  Backward returns the halo gradients to their owners and
    adds them to the edge rows (reference: ``shard_utils/halo.py:165-353``)."""

    @staticmethod
    def forward(ctx, x, dim, halo, edge_pad, group, sizes, periodic=False):
        n, r = _world(group), dist.get_rank(group=group)
        ctx.dim, ctx.halo, ctx.edge_pad, ctx.group, ctx.periodic = dim, halo, edge_pad, group, periodic
        ctx.sizes = tuple(sizes)
        ctx.extent = x.shape[dim]
        if halo == 0 and edge_pad == 0:
            ctx.trivial = True
            return x.clone()
        ctx.trivial = False
        parts = []
        from_left = from_right = None
        if halo > 0 and n > 1:
            def shape_of(k):
                s = list(x.shape)
                s[dim] = min(halo, k)
                return s

            has_left = periodic or r > 0
            has_right = periodic or r < n - 1
            send_left = x.narrow(dim, 0, min(halo, x.shape[dim])) if has_left else None
            send_right = x.narrow(dim, x.shape[dim] - min(halo, x.shape[dim]), min(halo, x.shape[dim])) if has_right else None
            from_left, from_right = _exchange_with_neighbours(
                send_left, send_right,
                shape_of(sizes[(r - 1) % n]) if has_left else None,
                shape_of(sizes[(r + 1) % n]) if has_right else None, group, x, periodic)
        ctx.left_w = from_left.shape[dim] if from_left is not None else 0
        ctx.right_w = from_right.shape[dim] if from_right is not None else 0

        def zeros(width):
            s = list(x.shape)
            s[dim] = width
            return x.new_zeros(s)

        ctx.left_pad = edge_pad if (from_left is None and edge_pad > 0) else 0
        ctx.right_pad = edge_pad if (from_right is None and edge_pad > 0) else 0
        if from_left is not None:
            parts.append(from_left)
        elif ctx.left_pad:
            parts.append(zeros(ctx.left_pad))
        parts.append(x)
        if from_right is not None:
            parts.append(from_right)
        elif ctx.right_pad:
            parts.append(zeros(ctx.right_pad))
        return torch.cat(parts, dim=dim)

    @staticmethod
    def backward(ctx, g):
        if ctx.trivial:
            return g, None, None, None, None, None, None
        dim = ctx.dim
        lw = ctx.left_w or ctx.left_pad
        rw = ctx.right_w or ctx.right_pad
        core = g.narrow(dim, lw, ctx.extent).clone()
        n, r = _world(ctx.group), dist.get_rank(group=ctx.group)
        if ctx.halo > 0 and n > 1:
            g_left = g.narrow(dim, 0, ctx.left_w) if ctx.left_w else None
            g_right = g.narrow(dim, g.shape[dim] - ctx.right_w, ctx.right_w) if ctx.right_w else None
            has_left = ctx.periodic or r > 0
            has_right = ctx.periodic or r < n - 1
            w = min(ctx.halo, ctx.extent)

            def shape_w():
                s = list(core.shape)
                s[dim] = w
                return s

            back_left, back_right = _exchange_with_neighbours(
                g_left, g_right, shape_w() if has_left else None, shape_w() if has_right else None,
                ctx.group, g, ctx.periodic)
            if back_left is not None:  # what my left neighbour computed on my first rows
                core.narrow(dim, 0, w).add_(back_left)
            if back_right is not None:
                core.narrow(dim, ctx.extent - w, w).add_(back_right)
        return core, None, None, None, None, None, None


class RingShift(torch.autograd.Function):
    """Send ``x`` to the next rank of the ring and return what the previous rank sent
    (shapes may differ per rank); the backward runs the ring the other way."""

    @staticmethod
    def forward(ctx, x, recv_shape, group, step=1):
        ctx.group, ctx.step, ctx.shape = group, step, tuple(x.shape)
        return _ring(x, recv_shape, group, step)

    @staticmethod
    def backward(ctx, g):
        return _ring(g, ctx.shape, ctx.group, -ctx.step), None, None, None


def _ring(x, recv_shape, group, step):
    n, r = _world(group), dist.get_rank(group=group)
    if n == 1:
        return x.clone()
    dst, src = (r + step) % n, (r - step) % n
    out = x.new_empty(recv_shape)
    ops = [dist.P2POp(dist.irecv, out, _global_rank(group, src), group=group),
           dist.P2POp(dist.isend, x.contiguous(), _global_rank(group, dst), group=group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return out


class AllToAllDims(torch.autograd.Function):
    """Move the shard from tensor dim ``src_dim`` to ``dst_dim`` (Shard(i) → Shard(j)) with one
    uneven all-to-all; the backward is the opposite move."""

    @staticmethod
    def forward(ctx, x, src_dim, dst_dim, src_sizes, dst_sizes, group):
        ctx.args = (src_dim, dst_dim, tuple(src_sizes), tuple(dst_sizes), group)
        return _a2a_dims(x, src_dim, dst_dim, src_sizes, dst_sizes, group)

    @staticmethod
    def backward(ctx, g):
        src_dim, dst_dim, src_sizes, dst_sizes, group = ctx.args
        return _a2a_dims(g, dst_dim, src_dim, dst_sizes, src_sizes, group), None, None, None, None, None


def _a2a_dims(x, src_dim, dst_dim, src_sizes, dst_sizes, group):
    """x is sharded on src_dim (this rank holds src_sizes[r]) and full on dst_dim; returns the
    tensor full on src_dim and sharded on dst_dim (this rank holds dst_sizes[r])."""
    n, r = _world(group), dist.get_rank(group=group)
    if n == 1:
        return x.clone()
    send = [t.contiguous() for t in torch.split(x, list(dst_sizes), dim=dst_dim)]
    recv = []
    for k in range(n):
        s = list(x.shape)
        s[src_dim] = src_sizes[k]
        s[dst_dim] = dst_sizes[r]
        recv.append(x.new_empty(s))
    _all_to_all(recv, send, group=group)
    return torch.cat(recv, dim=src_dim)
