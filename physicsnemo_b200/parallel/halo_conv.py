"""3×3 convolution of a height-sharded image with the halo exchange fused into the convolution kernel.

Reference behaviour: ``physicsnemo/domain_parallel/shard_utils/conv_patches.py`` + ``halo.py`` — before every
convolution each rank sends its boundary rows to its neighbours (point-to-point collectives), pads its shard with the
received rows, runs the library convolution and crops.  Here there is no separate exchange and no padded copy:

1. ``pnm_halo_publish`` copies the slab's first and last row into a small mailbox in symmetric (peer-mapped) memory
   and raises a flag in each neighbour's buffer;
2. ``pnm_conv2d_nhwc_halo`` — the tcgen05 implicit-GEMM convolution — computes the interior tiles first; tiles on the
   slab's first / last tile row fetch the missing input row straight from the neighbour's mailbox with plain
   (non-multicast) TMA loads once the flag has arrived, so the transfer overlaps the interior math.

Mailboxes are double-buffered by call parity; every wait on a flag is bounded (error word 6, ``PeerTimeoutError``).
The input gradient is the same operation on the output gradient with the flipped, transposed filter; the weight
gradient is local to the shard apart from the halo rows, which contribute through the rows received here.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as _g
from ..ops.conv import _pack_weight

_FLAG_BYTES = 256


class HaloConvRuntime:
    """Symmetric mailboxes + flags of one process group whose ranks hold consecutive height slabs (rank 0 on top)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, max_row_bytes: int = 1 << 22):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("HaloConvRuntime needs an initialised process group")
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.lib = _lib.load(required=True)
        vp, i, u = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint
        self.lib.pnm_halo_publish.argtypes = [vp, vp, vp, i, i, i, i, vp, vp, u, vp, vp]
        self.lib.pnm_conv2d_nhwc_halo.argtypes = [vp, vp, vp, i, i, i, i, i, vp, i, vp, vp, vp, vp, u, i, i, vp]
        self.lib.pnm_halo_publish.restype = self.lib.pnm_conv2d_nhwc_halo.restype = i
        self.row_bytes = (int(max_row_bytes) + 1023) // 1024 * 1024
        self.device = torch.device("cuda", torch.cuda.current_device())
        # [flags: from_up @0, from_down @4, block counter @8][slot 0: top, bottom][slot 1: top, bottom]
        self.buffer = symm.empty(_FLAG_BYTES + 4 * self.row_bytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        torch.cuda.synchronize()
        self.handle = symm.rendezvous(self.buffer, group=self.group.group_name)
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = 0
        dist.barrier(group=self.group)

    def _block(self, rank: int, slot: int, side: int) -> int:
        return self.bases[rank] + _FLAG_BYTES + (2 * slot + side) * self.row_bytes

    def conv3x3(self, x_nhwc: torch.Tensor, w_packed: torch.Tensor, bias: Optional[torch.Tensor], act: int = 0) -> torch.Tensor:
        """``x_nhwc``: this rank's slab ``[N, H_local, W, C]`` bf16 contiguous; returns ``[N, H_local, W, C_out]``."""
        n, h, w, c = x_nhwc.shape
        if h % 8 or c % 64 or w_packed.shape[1] != 9 * c:
            raise ValueError("halo convolution needs H_local % 8 == 0, C_in % 64 == 0 and a packed 3x3 filter")
        if n * w * c * 2 > self.row_bytes:
            raise ValueError(f"one boundary row ({n * w * c * 2} bytes) exceeds the mailbox ({self.row_bytes} bytes)")
        self.epoch += 1
        slot = self.epoch & 1
        up, down = self.rank - 1, self.rank + 1
        has_up, has_down = up >= 0, down < self.world
        st = torch.cuda.current_stream().cuda_stream
        me = self.bases[self.rank]
        err = self.lib.pnm_halo_publish(
            x_nhwc.data_ptr(), self._block(self.rank, slot, 0), self._block(self.rank, slot, 1), n, h, w, c,
            self.bases[up] + 4 if has_up else None,          # the upper neighbour waits on its "from_down" flag
            self.bases[down] + 0 if has_down else None,      # the lower neighbour waits on its "from_up" flag
            self.epoch, me + 8, st)
        if err:
            raise RuntimeError(f"pnm_halo_publish failed ({err})")
        y = torch.empty(n, h, w, w_packed.shape[0], dtype=torch.bfloat16, device=x_nhwc.device)
        b = None if bias is None else bias.detach().float().contiguous()
        err = self.lib.pnm_conv2d_nhwc_halo(
            x_nhwc.data_ptr(), w_packed.data_ptr(), y.data_ptr(), n, h, w, c, w_packed.shape[0],
            None if b is None else b.data_ptr(), act,
            self._block(up, slot, 1) if has_up else None,     # upper neighbour's bottom row
            self._block(down, slot, 0) if has_down else None,  # lower neighbour's top row
            me + 0, me + 4, self.epoch, 0, 0, st)
        if err:
            raise RuntimeError(f"pnm_conv2d_nhwc_halo failed ({err})")
        _g.launch_count += 2
        return y

    def check(self) -> None:
        from .peer import PeerTimeoutError

        code = self.lib.pnm_get_error()
        if code:
            raise PeerTimeoutError(f"device error word = {code} (6 = wait on a neighbour's halo flag ran out)")


class _HaloConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, rt: HaloConvRuntime):
        xh = x.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()
        y = rt.conv3x3(xh, _pack_weight(weight), bias)
        ctx.save_for_backward(xh, weight)
        ctx.rt, ctx.has_bias, ctx.x_dtype = rt, bias is not None, x.dtype
        return y.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        xh, weight = ctx.saved_tensors
        rt = ctx.rt
        dyh = dy.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            wt = weight.detach().flip(2, 3).transpose(0, 1)
            dx = rt.conv3x3(dyh, _pack_weight(wt), None).permute(0, 3, 1, 2).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            # weight gradient of the shard: the input rows just outside the slab pair with the slab's own dy rows, so the
            # shard needs its input padded by the neighbours' rows; fetch them with one small all-gather of boundary rows
            xp = _pad_with_neighbour_rows(xh, rt)
            dw = torch.nn.grad.conv2d_weight(xp.permute(0, 3, 1, 2), weight.shape, dyh.permute(0, 3, 1, 2), padding=(0, 1)).to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dyh.float().sum(dim=(0, 1, 2))
        return dx, dw, db, None


def _pad_with_neighbour_rows(xh: torch.Tensor, rt: HaloConvRuntime) -> torch.Tensor:
    """``[N, H+2, W, C]``: the slab with the neighbours' adjacent rows (zeros at the outer edges)."""
    rows = torch.stack([xh[:, 0], xh[:, -1]])                               # [2, N, W, C]
    gathered = [torch.empty_like(rows) for _ in range(rt.world)]
    dist.all_gather(gathered, rows, group=rt.group)
    zero = torch.zeros_like(xh[:, :1])
    above = gathered[rt.rank - 1][1].unsqueeze(1) if rt.rank > 0 else zero
    below = gathered[rt.rank + 1][0].unsqueeze(1) if rt.rank + 1 < rt.world else zero
    return torch.cat([above, xh, below], dim=1)


def halo_conv2d_3x3(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], runtime: HaloConvRuntime) -> torch.Tensor:
    """``conv2d(x_global, weight, bias, padding=1)`` restricted to this rank's height slab ``x [N, C, H_local, W]``.

    Returns an NCHW view of channels-last bf16 storage.  Gradients of the weight and bias are the shard's
    contributions: reduce them over the group like any data-parallel gradient.
    """
    return _HaloConv.apply(x, weight, bias, runtime)
