"""3×3 convolution of a height-sharded image with the halo exchange fused into the convolution kernels.

Reference behaviour: ``physicsnemo/domain_parallel/shard_utils/conv_patches.py`` + ``halo.py`` — before every
convolution each rank sends its boundary rows to its neighbours (point-to-point collectives), pads its shard with the
received rows, runs the library convolution and crops; the backward sends the halo gradients back and adds them.
Here there is no separate exchange and no padded copy:

1. ``pnm_halo_publish`` copies the slab's first and last row into a small mailbox in symmetric (peer-mapped) memory
   and raises a flag in each neighbour's buffer;
2. ``pnm_conv2d_nhwc_halo`` — the tcgen05 implicit-GEMM convolution — computes the interior tiles first; tiles on the
   slab's first / last tile row fetch the missing input row straight from the neighbour's mailbox with plain
   (non-multicast) TMA loads once the flag has arrived, so the transfer overlaps the interior math;
3. the two received rows are kept (a copy of ``2 · N · W · C`` values) for the weight gradient.

Backward: the input gradient is step 1 + 2 on the output gradient with the flipped, transposed filter (each rank
*pulls* the neighbours' gradient rows instead of receiving and adding halo gradients).  The weight gradient is the
library's split-reduction GEMM in convolution mode (``pnm_conv2d_wgrad_nhwc``), whose tap-shifted input boxes take
the rows above / below the slab from the copies made in step 3 — no collective, no library convolution.  The
bias gradient comes out of the same kernel.  Weight and bias gradients are per-shard partial sums: they are summed
over the group by the gradient reducer like any data-parallel gradient.

Mailboxes are double-buffered by call parity; every wait on a flag is bounded (error word 6, ``PeerTimeoutError``).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as _g
from ..ops.conv import _conv_dims, _cout_bwd, _pack_weight, _as_nhwc_bf16, unpack_wgrad

_FLAG_BYTES = 256


class HaloConvRuntime:
    """Symmetric mailboxes + flags of one process group whose ranks hold consecutive height slabs (rank 0 on top)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, max_row_bytes: int = 1 << 24, budget_s: float = 30.0):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("HaloConvRuntime needs an initialised process group")
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.lib = _lib.load(required=True)
        vp, i, u, d = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_double
        self.lib.pnm_halo_publish.argtypes = [vp, vp, vp, i, i, i, i, vp, vp, u, vp, vp]
        self.lib.pnm_conv2d_nhwc_halo.argtypes = [vp, vp, vp, i, i, i, i, i, vp, i, vp, vp, vp, vp, u, i, i, vp, d]
        self.lib.pnm_conv2d_wgrad_nhwc.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp, vp, vp, vp, u, d, i, vp]
        self.lib.pnm_halo_publish.restype = self.lib.pnm_conv2d_nhwc_halo.restype = self.lib.pnm_conv2d_wgrad_nhwc.restype = i
        self.row_bytes = (int(max_row_bytes) + 1023) // 1024 * 1024
        self.device = torch.device("cuda", torch.cuda.current_device())
        # [flags: from_up @0, from_down @4, block counter @8][slot 0: top, bottom][slot 1: top, bottom]
        self.buffer = symm.empty(_FLAG_BYTES + 4 * self.row_bytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        torch.cuda.synchronize()
        self.handle = symm.rendezvous(self.buffer, group=self.group.group_name)
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = 0
        self.budget_s = float(budget_s)
        self.loopback = False   # measurement aid: treat the slab as a whole image (zero padding, no neighbour reads)
        from .peer import register_loopback

        register_loopback(self)
        dist.barrier(group=self.group)

    def _block(self, rank: int, slot: int, side: int) -> int:
        return self.bases[rank] + _FLAG_BYTES + (2 * slot + side) * self.row_bytes

    def fits(self, n: int, h: int, w: int, c: int) -> bool:
        return h % 8 == 0 and c % 64 == 0 and n * w * c * 2 <= self.row_bytes

    def conv3x3(self, x_nhwc: torch.Tensor, w_packed: torch.Tensor, bias: Optional[torch.Tensor], act: int = 0,
                keep_rows: bool = False):
        """``x_nhwc``: this rank's slab ``[N, H_local, W, C]`` bf16 contiguous; returns ``[N, H_local, W, C_out]``
        (and, with ``keep_rows``, copies of the rows received from above / below — ``None`` at the outer edges)."""
        n, h, w, c = x_nhwc.shape
        if h % 8 or c % 64 or w_packed.shape[1] != 9 * c:
            raise ValueError("halo convolution needs H_local % 8 == 0, C_in % 64 == 0 and a packed 3x3 filter")
        if n * w * c * 2 > self.row_bytes:
            raise ValueError(f"one boundary row ({n * w * c * 2} bytes) exceeds the mailbox ({self.row_bytes} bytes)")
        self.epoch += 1
        slot = self.epoch & 1
        up, down = self.rank - 1, self.rank + 1
        has_up, has_down = up >= 0 and not self.loopback, down < self.world and not self.loopback
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
        if b is not None and b.numel() != w_packed.shape[0]:
            b = torch.nn.functional.pad(b, (0, w_packed.shape[0] - b.numel()))
        up_ptr = self._block(up, slot, 1) if has_up else None       # upper neighbour's bottom row
        down_ptr = self._block(down, slot, 0) if has_down else None  # lower neighbour's top row
        err = self.lib.pnm_conv2d_nhwc_halo(
            x_nhwc.data_ptr(), w_packed.data_ptr(), y.data_ptr(), n, h, w, c, w_packed.shape[0],
            None if b is None else b.data_ptr(), act, up_ptr, down_ptr, me + 0, me + 4, self.epoch, 0, 0, st, self.budget_s)
        if err:
            raise RuntimeError(f"pnm_conv2d_nhwc_halo failed ({err})")
        _g.launch_count += 2
        if not keep_rows:
            return y
        # the convolution kernel has seen both flags, so the rows are complete; the neighbour cannot overwrite this
        # mailbox slot before it has seen this rank's NEXT publish, which is enqueued after these copies
        rows = []
        for ptr in (up_ptr, down_ptr):
            if ptr is None:
                rows.append(None)
                continue
            r = torch.empty(n, 1, w, c, dtype=torch.bfloat16, device=x_nhwc.device)
            self._copy_from_address(r, ptr)
            rows.append(r)
        return y, rows[0], rows[1]

    def wgrad3x3(self, dy_nhwc: torch.Tensor, x_nhwc: torch.Tensor, up_row, down_row, want_bias: bool):
        """Shard's contribution to ``dW [Cout, 9*Cin]`` (fp32, tap-major) and ``db``: one split-reduction kernel."""
        n, h, w, cin = x_nhwc.shape
        cout = dy_nhwc.shape[-1]
        dw = torch.zeros(cout, 9 * cin, dtype=torch.float32, device=x_nhwc.device)
        db = torch.zeros(cout, dtype=torch.float32, device=x_nhwc.device) if want_bias else None
        err = self.lib.pnm_conv2d_wgrad_nhwc(
            dy_nhwc.data_ptr(), x_nhwc.data_ptr(), dw.data_ptr(), None if db is None else db.data_ptr(), n, h, w, cin, cout,
            None if up_row is None else up_row.data_ptr(), None if down_row is None else down_row.data_ptr(), None, None,
            0, self.budget_s, 0, torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_conv2d_wgrad_nhwc failed ({err})")
        _g.launch_count += 1
        return dw, db

    def _copy_from_address(self, dst: torch.Tensor, src_ptr: int) -> None:
        """Copy from a peer-mapped address into ``dst`` with the library's own vector-load kernel (no flag wait)."""
        from .peer import _declare

        _declare(self.lib)
        own = (ctypes.c_void_p * 1)(self.bases[self.rank])
        err = self.lib.pnm_peer_pull(src_ptr, dst.data_ptr(), dst.numel() * dst.element_size(), -1, own, 0, 1, 0, 0, 1.0,
                                     torch.cuda.current_stream().cuda_stream, None, 16)
        if err:
            raise RuntimeError(f"pnm_peer_pull failed ({err})")
        _g.launch_count += 1

    def check(self) -> None:
        from .peer import PeerTimeoutError

        code = self.lib.pnm_get_error()
        if code:
            raise PeerTimeoutError(f"device error word = {code} (6 = wait on a neighbour's halo flag ran out)")


_halo_runtimes: Dict[str, HaloConvRuntime] = {}


def get_halo_runtime(group: Optional[dist.ProcessGroup] = None) -> HaloConvRuntime:
    g = group if group is not None else dist.group.WORLD
    rt = _halo_runtimes.get(g.group_name)
    if rt is None:
        rt = HaloConvRuntime(g)
        _halo_runtimes[g.group_name] = rt
    return rt


class _HaloConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, rt: HaloConvRuntime):
        cin_p, cout_p = _conv_dims(weight)
        xh = _as_nhwc_bf16(x, cin_p)
        need_w = weight.requires_grad or (bias is not None and bias.requires_grad)
        res = rt.conv3x3(xh, _pack_weight(weight, cin_p, cout_p), bias, keep_rows=need_w)
        y, up_row, down_row = res if need_w else (res, None, None)
        ctx.save_for_backward(xh, weight, up_row, down_row)
        ctx.rt, ctx.has_bias, ctx.x_dtype = rt, bias is not None, x.dtype
        if cout_p != weight.shape[0]:
            y = y[..., :weight.shape[0]]
        return y.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        xh, weight, up_row, down_row = ctx.saved_tensors
        rt = ctx.rt
        cout, cin = weight.shape[:2]
        cin_p, _ = _conv_dims(weight)
        cout_p = _cout_bwd(weight)
        dyh = _as_nhwc_bf16(dy, cout_p)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            wt = weight.detach().flip(2, 3).transpose(0, 1)
            dxh = rt.conv3x3(dyh, _pack_weight(wt, cout_p, cin_p), None)
            dx = dxh[..., :cin].permute(0, 3, 1, 2).to(ctx.x_dtype)
        need_w, need_b = ctx.needs_input_grad[1], ctx.has_bias and ctx.needs_input_grad[2]
        if need_w or need_b:
            dwp, dbp = rt.wgrad3x3(dyh, xh, up_row, down_row, need_b)
            if need_w:
                dw = unpack_wgrad(dwp, weight, cin_p)
            if need_b:
                db = dbp[:cout]
        return dx, dw, db, None


def halo_conv_supported(x_local: torch.Tensor, weight: torch.Tensor, rt: Optional[HaloConvRuntime] = None) -> bool:
    """The fused path covers 3×3, stride 1, padding 1 convolutions of CUDA slabs with ``H_local % 8 == 0``."""
    if not (x_local.is_cuda and x_local.dim() == 4 and weight.dim() == 4 and tuple(weight.shape[2:]) == (3, 3)):
        return False
    n, _, h, w = x_local.shape
    cin_p, _ = _conv_dims(weight)
    cout_p = _cout_bwd(weight)
    if cin_p > 4 * weight.shape[1] or h % 8:
        return False
    row = n * w * max(cin_p, cout_p) * 2
    return rt is None or row <= rt.row_bytes


def halo_conv2d_3x3(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], runtime: HaloConvRuntime) -> torch.Tensor:
    """``conv2d(x_global, weight, bias, padding=1)`` restricted to this rank's height slab ``x [N, C, H_local, W]``.

    Returns an NCHW view of channels-last bf16 storage.  Gradients of the weight and bias are the shard's
    contributions: reduce them over the group like any data-parallel gradient.
    """
    return _HaloConv.apply(x, weight, bias, runtime)
