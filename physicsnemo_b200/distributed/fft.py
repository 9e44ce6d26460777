"""Distributed 2-D real FFT by pencil transposition over the group ``"spatial_parallel"``.

Parity: ``physicsnemo/distributed/fft.py`` — ``conj_pad_helper_2d`` (``:31-63``),
``DistributedRFFT2`` (``:66-152``), ``DistributedIRFFT2`` (``:155-244``): local FFT along
``dim[0]`` → all-to-all transpose → FFT along ``dim[1]`` → truncate to ``n//2+1``; the inverse
pads conjugate-symmetrically first.
"""
import torch
import torch.distributed as dist

from .manager import DistributedManager
from .mappings import gather_from_parallel_region, scatter_to_parallel_region
from .utils import distributed_transpose, pad_helper, truncate_helper


def conj_pad_helper_2d(tensor, pad_dim, other_dim, new_size):
    """Hermitian continuation along ``pad_dim`` (needs the reversed ``other_dim``, hence gather → flip → scatter)."""
    ndim = tensor.ndim
    pad_dim = (pad_dim + ndim) % ndim
    other_dim = (other_dim + ndim) % ndim
    orig_size = tensor.shape[pad_dim]
    tensor_pad = pad_helper(tensor, pad_dim, new_size, mode="conj")
    tensor_pad_gather = gather_from_parallel_region(tensor_pad, other_dim, None, "spatial_parallel") \
        if False else _gather_equal(tensor_pad, other_dim)
    flip_slice = [slice(0, x) if i != pad_dim else slice(orig_size, new_size) for i, x in enumerate(tensor_pad_gather.shape)]
    tensor_pad_gather[flip_slice] = torch.flip(tensor_pad_gather[flip_slice], dims=[other_dim]).roll(shifts=1, dims=[other_dim])
    return scatter_to_parallel_region(tensor_pad_gather, other_dim, "spatial_parallel")


def _gather_equal(t, dim):
    group = DistributedManager().group("spatial_parallel")
    n = dist.get_world_size(group=group)
    outs = [torch.empty_like(t) for _ in range(n)]
    dist.all_gather(outs, t.contiguous(), group=group)
    return torch.cat(outs, dim=dim)


class DistributedRFFT2(torch.autograd.Function):
    """``rfft2`` of a tensor sharded along ``dim[1]``; the result is sharded along ``dim[0]``."""

    @staticmethod
    def forward(ctx, x, s, dim, norm="ortho"):
        ctx.s, ctx.dim, ctx.norm = s, dim, norm
        group = DistributedManager().group("spatial_parallel")
        x1 = torch.fft.fft(x, n=s[0], dim=dim[0], norm=norm)
        x1_recv, _ = distributed_transpose(x1, dim[0], dim[1], group=group, async_op=False)
        x1_tran = torch.cat(x1_recv, dim=dim[1])
        x2 = torch.fft.fft(x1_tran, n=s[1], dim=dim[1], norm=norm)
        ctx.last_dim_size = x2.shape[dim[1]]
        return truncate_helper(x2, dim[1], x2.shape[dim[1]] // 2 + 1)

    @staticmethod
    def backward(ctx, grad_output):
        dim, norm = ctx.dim, ctx.norm
        group = DistributedManager().group("spatial_parallel")
        g_pad = pad_helper(grad_output, dim[1], ctx.last_dim_size, mode="zero")
        g1 = torch.fft.ifft(g_pad, dim=dim[1], norm=norm)
        g1_recv, _ = distributed_transpose(g1, dim[1], dim[0], group=group, async_op=False)
        g1_tran = torch.cat(g1_recv, dim=dim[0])
        gx = torch.real(torch.fft.ifft(g1_tran, dim=dim[0], norm=norm))
        return gx, None, None, None


class DistributedIRFFT2(torch.autograd.Function):
    """Inverse of ``DistributedRFFT2``."""

    @staticmethod
    def forward(ctx, x, s, dim, norm="ortho"):
        ctx.s, ctx.dim, ctx.norm = s, dim, norm
        ctx.orig_dim_size = x.shape[dim[1]]
        group = DistributedManager().group("spatial_parallel")
        if s is not None:
            first_dim_size, last_dim_size = s[0], s[1]
            ctx.last_dim_size = last_dim_size
        else:
            first_dim_size = x.shape[dim[0]] * dist.get_world_size(group=group)
            last_dim_size = 2 * (x.shape[dim[1]] - 1)
        x_pad = conj_pad_helper_2d(x, dim[1], dim[0], last_dim_size)
        x1 = torch.fft.ifft(x_pad, n=last_dim_size, dim=dim[1], norm=norm)
        x1_recv, _ = distributed_transpose(x1, dim[1], dim[0], group=group, async_op=False)
        x1_tran = torch.cat(x1_recv, dim=dim[0])
        x2 = torch.fft.ifft(x1_tran, n=first_dim_size, dim=dim[0], norm=norm)
        return torch.real(x2)

    @staticmethod
    def backward(ctx, grad_output):
        dim, norm = ctx.dim, ctx.norm
        group = DistributedManager().group("spatial_parallel")
        g1 = torch.fft.fft(grad_output, dim=dim[0], norm=norm)
        g1_recv, _ = distributed_transpose(g1, dim[0], dim[1], group=group, async_op=False)
        g1_tran = torch.cat(g1_recv, dim=dim[1])
        g2 = torch.fft.fft(g1_tran, dim=dim[1], norm=norm)
        return truncate_helper(g2, dim[1], ctx.orig_dim_size), None, None, None
