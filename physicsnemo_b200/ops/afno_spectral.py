"""AFNO spectral filter on the library's Fourier kernels, with the token ↔ channel resharding fused in (``csrc/afno_spectral.cu``).

``afno_filter(tokens, w1, b1, w2, b2, ...)`` computes, for the channel blocks this rank owns,
``irfft2(softshrink(blockMLP(rfft2(x)[kept modes])))`` (``ortho`` norm) of the global token tensor ``x[B, H, W, C]`` that
is sharded over the ranks by tokens: the row kernels pull the channel slices of the tokens from their owners and push
the filtered slices back, so the all-to-alls of a token ↔ channel transpose never exist as separate steps
(reference: ``physicsnemo/nn/module/afno_layers.py:187-327`` on ``torch.fft`` + eight real einsums; its distributed
variant gathers channels and all-reduces, ``physicsnemo/models/afno/distributed/layers.py:222-244``).

With one rank (``exchange=None``) the same kernels run on local buffers; that path is the single-GPU AFNO filter.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from . import gemm as _g


def _lib_af():
    lib = _lib.load(required=True)
    if not getattr(lib, "_afno_declared", False):
        c = ctypes
        vp, i, u, ll, f, d = c.c_void_p, c.c_int, c.c_uint, c.c_longlong, c.c_float, c.c_double
        lib.pnm_afno_rows_r2c.argtypes = [vp, vp, vp, ll, i, i, vp, i, i, u, ll, d, vp, vp]
        lib.pnm_afno_rows_c2r.argtypes = [vp, vp, vp, ll, i, i, vp, i, i, u, ll, vp, vp, vp]
        lib.pnm_afno_cols_fwd.argtypes = [vp] * 9 + [i, vp, f, vp]
        lib.pnm_afno_cols_bwd.argtypes = [vp] * 11 + [i, vp, vp]
        for n in ("pnm_afno_rows_r2c", "pnm_afno_rows_c2r", "pnm_afno_cols_fwd", "pnm_afno_cols_bwd"):
            getattr(lib, n).restype = i
        lib._afno_declared = True
    return lib


def _factor(n: int):
    """``(n1, n2)`` with ``n1 * n2 == n`` and the factors as close as possible (two-level transform along H)."""
    best = (1, n)
    for a in range(1, int(n ** 0.5) + 1):
        if n % a == 0:
            best = (a, n // a)
    return best


class FilterGeometry:
    """Shapes of one filter call: token grid, channel blocks, the blocks this rank owns."""

    def __init__(self, B: int, H: int, W: int, C: int, num_blocks: int, kept: int, rank: int = 0, world: int = 1):
        if num_blocks % world or (B * H * W) % world:
            raise ValueError("the channel blocks and the tokens must divide evenly over the ranks")
        self.B, self.H, self.W, self.C = B, H, W, C
        self.Cb = C // num_blocks
        self.nb = num_blocks
        self.KX = min(kept, W // 2)
        self.nblk = num_blocks // world
        self.blk0 = rank * self.nblk
        self.Tp = B * H * W // world
        self.H1, self.H2 = _factor(H)
        self.rank, self.world = rank, world
        self.arr = (ctypes.c_int * 10)(B, H, W, C, self.Cb, self.KX, self.blk0, self.nblk, self.H1, self.H2)

    def supported(self) -> bool:
        return self.Cb % 8 == 0 and self.Cb <= 128 and 2 * self.KX <= self.W and self.H * self.Cb * 8 * 3 + self.H * 8 <= 220 * 1024


def _ptrs8(ptrs):
    ptrs = list(ptrs)
    ptrs = ptrs + [ptrs[0]] * (8 - len(ptrs))
    return (ctypes.c_void_p * 8)(*ptrs)


class _AfnoFilterFn(torch.autograd.Function):
    """tokens [Tp, C] bf16 (this rank's tokens, all channels) -> filtered tokens [Tp, C] bf16."""

    @staticmethod
    def forward(ctx, tokens, w1, b1, w2, b2, geo: FilterGeometry, lam: float, exchange):
        lib = _lib_af()
        dev = tokens.device
        st = torch.cuda.current_stream().cuda_stream
        g = geo
        rows, ld = g.B * g.H, g.nblk * g.Cb
        Y = torch.empty(rows, g.KX, ld, 2, dtype=torch.float32, device=dev)
        Y2 = torch.empty_like(Y)
        sv = [torch.empty(g.B * g.KX, g.nblk, g.H, g.Cb, 2, dtype=torch.float32, device=dev) for _ in range(3)]
        w1f, b1f, w2f, b2f = (t.detach().float().contiguous() for t in (w1, b1, w2, b2))
        if exchange is None:
            src = tokens.contiguous()
            out = torch.empty_like(src)
            rc = lib.pnm_afno_rows_r2c(_ptrs8([src.data_ptr()]), Y.data_ptr(), g.arr, g.Tp, 0, 0, None, 0, 1, 0, 0, 1.0, None, st)
            _g._check(rc, "pnm_afno_rows_r2c")
            rc = lib.pnm_afno_cols_fwd(Y.data_ptr(), Y2.data_ptr(), sv[0].data_ptr(), sv[1].data_ptr(), sv[2].data_ptr(),
                                       w1f.data_ptr(), b1f.data_ptr(), w2f.data_ptr(), b2f.data_ptr(), g.nb, g.arr, float(lam), st)
            _g._check(rc, "pnm_afno_cols_fwd")
            rc = lib.pnm_afno_rows_c2r(Y2.data_ptr(), _ptrs8([out.data_ptr()]), g.arr, g.Tp, 1, 0, None, 0, 1, 0, 0, None, None, st)
            _g._check(rc, "pnm_afno_rows_c2r")
        else:
            out = exchange.transform(lib, tokens, Y, Y2, lambda: _cols_fwd(lib, Y, Y2, sv, w1f, b1f, w2f, b2f, g, lam, st), g,
                                     kw_in=0, kw_out=1)
        _g.launch_count += 3
        ctx.save_for_backward(w1f, w2f, *sv)
        ctx.geo, ctx.exchange = geo, exchange
        ctx.dtypes = (w1.dtype, b1.dtype, w2.dtype, b2.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        lib = _lib_af()
        w1f, w2f, Z, O1, O2 = ctx.saved_tensors
        g, exchange = ctx.geo, ctx.exchange
        dev = dout.device
        st = torch.cuda.current_stream().cuda_stream
        rows, ld = g.B * g.H, g.nblk * g.Cb
        dY2 = torch.empty(rows, g.KX, ld, 2, dtype=torch.float32, device=dev)
        dY = torch.empty_like(dY2)
        dw1 = torch.zeros(2, g.nb, g.Cb, g.Cb, dtype=torch.float32, device=dev)
        dw2 = torch.zeros_like(dw1)
        db1 = torch.zeros(2, g.nb, g.Cb, dtype=torch.float32, device=dev)
        db2 = torch.zeros_like(db1)

        def cols():
            rc = lib.pnm_afno_cols_bwd(dY2.data_ptr(), dY.data_ptr(), Z.data_ptr(), O1.data_ptr(), O2.data_ptr(), w1f.data_ptr(),
                                       w2f.data_ptr(), dw1.data_ptr(), db1.data_ptr(), dw2.data_ptr(), db2.data_ptr(), g.nb, g.arr, st)
            _g._check(rc, "pnm_afno_cols_bwd")

        d = dout.to(torch.bfloat16).contiguous()
        if exchange is None:
            dx = torch.empty_like(d)
            # adjoint of the weighted c2r = r2c with the same weights; adjoint of the r2c = unweighted c2r
            rc = lib.pnm_afno_rows_r2c(_ptrs8([d.data_ptr()]), dY2.data_ptr(), g.arr, g.Tp, 1, 0, None, 0, 1, 0, 0, 1.0, None, st)
            _g._check(rc, "pnm_afno_rows_r2c")
            cols()
            rc = lib.pnm_afno_rows_c2r(dY.data_ptr(), _ptrs8([dx.data_ptr()]), g.arr, g.Tp, 0, 0, None, 0, 1, 0, 0, None, None, st)
            _g._check(rc, "pnm_afno_rows_c2r")
        else:
            dx = exchange.transform(lib, d, dY2, dY, cols, g, kw_in=1, kw_out=0)
        _g.launch_count += 3
        dt = ctx.dtypes
        return dx, dw1.to(dt[0]), db1.to(dt[1]), dw2.to(dt[2]), db2.to(dt[3]), None, None, None


def _cols_fwd(lib, Y, Y2, sv, w1f, b1f, w2f, b2f, g, lam, st):
    rc = lib.pnm_afno_cols_fwd(Y.data_ptr(), Y2.data_ptr(), sv[0].data_ptr(), sv[1].data_ptr(), sv[2].data_ptr(), w1f.data_ptr(),
                               b1f.data_ptr(), w2f.data_ptr(), b2f.data_ptr(), g.nb, g.arr, float(lam), st)
    _g._check(rc, "pnm_afno_cols_fwd")


class TokenChannelExchange:
    """Symmetric token buffers of a group of ranks for ``afno_filter``: ``src`` (read by the peers' row kernels) and
    ``dst`` (written by the peers' inverse row kernels), plus the flags that order the two transfers."""

    def __init__(self, group, tokens_per_rank: int, channels: int):
        from ..parallel.peer import PeerRegions

        floats = tokens_per_rank * channels // 2 + 64
        self.regions = PeerRegions(group, region_floats=floats, n_regions=2)
        self.rt = self.regions.rt
        self.world, self.rank = self.rt.world, self.rt.rank
        self.counter = torch.zeros(4, dtype=torch.int32, device=self.rt.device)
        self.lib_peer = None

    def transform(self, lib, tokens, Yin, Yout, cols_fn, g: FilterGeometry, kw_in: int, kw_out: int):
        rt = self.rt
        st = torch.cuda.current_stream().cuda_stream
        n = tokens.numel()
        src_view, src_ptrs = self.regions.region(n // 2, tokens.device)
        dst_view, dst_ptrs = self.regions.region(n // 2, tokens.device)
        src_view.view(torch.bfloat16)[:n].view_as(tokens).copy_(tokens)       # publish this rank's tokens
        peer = self.regions.publish()
        bases, rank, world, ep, cap, budget, ebase = peer
        if len(src_ptrs) != g.world:                                          # loopback: every "peer" is this rank
            src_ptrs, dst_ptrs = src_ptrs * g.world, dst_ptrs * g.world
        rc = lib.pnm_afno_rows_r2c(_ptrs8(src_ptrs), Yin.data_ptr(), g.arr, g.Tp, kw_in, 1, bases, rank, world, ep, cap, budget,
                                   ebase, st)
        _g._check(rc, "pnm_afno_rows_r2c")
        cols_fn()
        epoch2 = rt.next_epoch()
        bases, rank, world, ep2, cap, budget, ebase = rt.peer_args(epoch2)
        rc = lib.pnm_afno_rows_c2r(Yout.data_ptr(), _ptrs8(dst_ptrs), g.arr, g.Tp, kw_out, 1, bases, rank, world, ep2, cap, ebase,
                                   self.counter.data_ptr(), st)
        _g._check(rc, "pnm_afno_rows_c2r")
        # every rank's slices have landed in this rank's dst buffer once all flags of the second call are up
        out = torch.empty_like(tokens)
        rt.pull(dst_ptrs[rt.rank if len(set(dst_ptrs)) > 1 else 0], out, n * 2, epoch2, flag_from=-2)
        return out

    def step_done(self):
        self.regions.step_done()


def afno_filter(tokens: torch.Tensor, w1, b1, w2, b2, geo: FilterGeometry, sparsity_threshold: float,
                exchange: Optional[TokenChannelExchange] = None) -> torch.Tensor:
    """Filtered tokens (without the layer's residual): ``tokens`` is this rank's ``[Tp, C]`` bf16 slice of the token tensor."""
    return _AfnoFilterFn.apply(tokens, w1, b1, w2, b2, geo, float(sparsity_threshold), exchange)
