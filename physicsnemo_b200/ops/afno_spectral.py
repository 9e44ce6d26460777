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
        lib.pnm_afno_rows_c2r_add.argtypes = [vp, vp, vp, vp, vp, ll, i, vp]
        lib.pnm_afno_cols_fwd.argtypes = [vp] * 9 + [i, vp, f, vp]
        lib.pnm_afno_cols_bwd.argtypes = [vp] * 11 + [i, vp, vp]
        lib.pnm_afno_cols_dft.argtypes = [vp, vp, vp, vp, i, f, vp]
        lib.pnm_afno_cols_idft.argtypes = [vp, vp, vp, i, f, vp]
        for n in ("pnm_afno_rows_r2c", "pnm_afno_rows_c2r", "pnm_afno_rows_c2r_add", "pnm_afno_cols_fwd", "pnm_afno_cols_bwd", "pnm_afno_cols_dft",
                  "pnm_afno_cols_idft"):
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
        self.Mb = B * self.KX * H                       # spectral rows (b, kx, ky) of one channel block
        self.Mp = -(-self.Mb // 128) * 128              # ... padded to the GEMM's M tile

    def supported(self) -> bool:
        return self.Cb % 8 == 0 and self.Cb <= 128 and 2 * self.KX <= self.W and self.H * self.Cb * 8 * 3 + self.H * 8 <= 220 * 1024


def _ptrs8(ptrs):
    ptrs = list(ptrs)
    ptrs = ptrs + [ptrs[0]] * (8 - len(ptrs))
    return (ctypes.c_void_p * 8)(*ptrs)


def _expand_weight(w: torch.Tensor) -> torch.Tensor:
    """Complex block weights ``w[2, nb, Cb_in, Cb_out]`` as the real matrices ``[nb, 2 Cb (out), 2 Cb (in)]`` (bf16) that
    act on ``[real | imag]`` rows: ``[xr | xi] @ [[wr, wi], [-wi, wr]]``, stored output-major for ``gemm_tn``."""
    wr, wi = w[0].transpose(1, 2), w[1].transpose(1, 2)
    top = torch.cat([wr, -wi], dim=2)
    bottom = torch.cat([wi, wr], dim=2)
    return torch.cat([top, bottom], dim=1).to(torch.bfloat16).contiguous()


def _fold_weight_grad(dwe: torch.Tensor, cb: int) -> torch.Tensor:
    """Inverse of ``_expand_weight`` for gradients: ``[nb, 2 Cb, 2 Cb]`` fp32 -> ``[2, nb, Cb_in, Cb_out]``."""
    a, b, c, d = dwe[:, :cb, :cb], dwe[:, :cb, cb:], dwe[:, cb:, :cb], dwe[:, cb:, cb:]
    return torch.stack([(a + d).transpose(1, 2), (c - b).transpose(1, 2)])


class _AfnoFilterTcFn(torch.autograd.Function):
    """The filter with its block MLP on the tensor cores: Fourier kernels write / read the ``[real | imag]`` bf16
    expansion of the spectrum, the two complex layers are ``gemm_tn`` calls with bias / ReLU epilogues, their backward
    ``gemm_nt`` (weight and bias gradients in one pass) and ``gemm_tn`` with the ReLU mask in the epilogue."""

    @staticmethod
    def forward(ctx, tokens, w1, b1, w2, b2, geo: FilterGeometry, lam: float, exchange, add_input=False, residual=None):
        lib = _lib_af()
        dev = tokens.device
        st = torch.cuda.current_stream().cuda_stream
        g = geo
        rows, ld, cb2 = g.B * g.H, g.nblk * g.Cb, 2 * g.Cb
        own = slice(g.blk0, g.blk0 + g.nblk)
        Y = torch.empty(rows, g.KX, ld, 2, dtype=torch.float32, device=dev)
        Y2 = torch.empty_like(Y)
        Z = torch.empty(g.nblk, g.Mp, cb2, dtype=torch.bfloat16, device=dev)
        if g.Mp > g.Mb:
            Z[:, g.Mb:].zero_()                                   # rows that pad a block to the GEMM's M tile
        O1, O2 = torch.empty_like(Z), torch.empty_like(Z)
        w1e, w2e = _expand_weight(w1.detach()[:, own]), _expand_weight(w2.detach()[:, own])
        b1e = torch.cat([b1.detach()[0, own], b1.detach()[1, own]], dim=1).float().contiguous()
        b2e = torch.cat([b2.detach()[0, own], b2.detach()[1, own]], dim=1).float().contiguous()

        def cols():
            _g._check(lib.pnm_afno_cols_dft(Y.data_ptr(), Z.data_ptr(), None, g.arr, g.Mp, 0.0, st), "pnm_afno_cols_dft")
            _g.gemm_tn_stacked(Z, w1e, bias=b1e, act=_g.ACT_RELU, out=O1)            # all blocks in one launch
            _g.gemm_tn_stacked(O1, w2e, bias=b2e, out=O2)
            _g._check(lib.pnm_afno_cols_idft(O2.data_ptr(), Y2.data_ptr(), g.arr, g.Mp, float(lam), st), "pnm_afno_cols_idft")

        if exchange is None:
            src = tokens.contiguous()
            out = torch.empty_like(src)
            rc = lib.pnm_afno_rows_r2c(_ptrs8([src.data_ptr()]), Y.data_ptr(), g.arr, g.Tp, 0, 0, None, 0, 1, 0, 0, 1.0, None, st)
            _g._check(rc, "pnm_afno_rows_r2c")
            cols()
            addends = ([src] if add_input else []) + ([residual.contiguous()] if residual is not None else [])
            _rows_c2r_local(lib, Y2, out, addends, g, 1, st)
        else:
            if add_input or residual is not None:
                raise ValueError("residual terms are fused only on the single-GPU path")
            out = exchange.transform(lib, tokens, Y, Y2, cols, g, kw_in=0, kw_out=1)
        _g.launch_count += 4
        ctx.save_for_backward(w1e, w2e, Z, O1, O2)
        ctx.geo, ctx.exchange, ctx.lam = geo, exchange, float(lam)
        ctx.add_input, ctx.has_residual = bool(add_input), residual is not None
        ctx.dtypes = (w1.dtype, b1.dtype, w2.dtype, b2.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        lib = _lib_af()
        w1e, w2e, Z, O1, O2 = ctx.saved_tensors
        g, exchange, lam = ctx.geo, ctx.exchange, ctx.lam
        dev = dout.device
        st = torch.cuda.current_stream().cuda_stream
        rows, ld, cb2 = g.B * g.H, g.nblk * g.Cb, 2 * g.Cb
        dY2 = torch.empty(rows, g.KX, ld, 2, dtype=torch.float32, device=dev)
        dY = torch.empty_like(dY2)
        G2 = torch.empty_like(Z)
        if g.Mp > g.Mb:
            G2[:, g.Mb:].zero_()          # zero padding rows: they then contribute nothing to the weight gradients
        G1, dZ = torch.empty_like(Z), torch.empty_like(Z)
        # the four accumulators of the weight / bias gradients as views of ONE zero-filled buffer (one fill kernel, not four)
        nw, nbias = g.nblk * cb2 * cb2, g.nblk * cb2
        acc = torch.zeros(2 * nw + 2 * nbias, dtype=torch.float32, device=dev)
        dw1e, dw2e = acc[:nw].view(g.nblk, cb2, cb2), acc[nw:2 * nw].view(g.nblk, cb2, cb2)
        db1e, db2e = acc[2 * nw:2 * nw + nbias].view(g.nblk, cb2), acc[2 * nw + nbias:].view(g.nblk, cb2)
        w1t, w2t = w1e.transpose(1, 2).contiguous(), w2e.transpose(1, 2).contiguous()

        def cols():
            # adjoint of the inverse transform is the forward one; the soft-shrink mask comes from the saved O2
            _g._check(lib.pnm_afno_cols_dft(dY2.data_ptr(), G2.data_ptr(), O2.data_ptr(), g.arr, g.Mp, lam, st), "pnm_afno_cols_dft")
            _g.gemm_nt_stacked(G2, O1, dw2e, db2e)
            _g.gemm_tn_stacked(G2, w2t, aux=O1, aux_mode=_g.AUX_DRELU, out=G1)
            _g.gemm_nt_stacked(G1, Z, dw1e, db1e)
            _g.gemm_tn_stacked(G1, w1t, out=dZ)
            _g._check(lib.pnm_afno_cols_idft(dZ.data_ptr(), dY.data_ptr(), g.arr, g.Mp, 0.0, st), "pnm_afno_cols_idft")

        d = dout.to(torch.bfloat16).contiguous()
        if exchange is None:
            dx = torch.empty_like(d)
            rc = lib.pnm_afno_rows_r2c(_ptrs8([d.data_ptr()]), dY2.data_ptr(), g.arr, g.Tp, 1, 0, None, 0, 1, 0, 0, 1.0, None, st)
            _g._check(rc, "pnm_afno_rows_r2c")
            cols()
            # the input's own residual path: its gradient is the incoming one, added in the same store
            _rows_c2r_local(lib, dY, dx, [d] if ctx.add_input else [], g, 0, st)
        else:
            dx = exchange.transform(lib, d, dY2, dY, cols, g, kw_in=1, kw_out=0)
        _g.launch_count += 4
        dt = ctx.dtypes
        own = slice(g.blk0, g.blk0 + g.nblk)

        def scatter(part, shape, dtype):
            if g.nblk == g.nb:                       # this rank owns every block: nothing to embed
                return part.to(dtype)
            full = torch.zeros(shape, dtype=torch.float32, device=dev)
            full[:, own] = part
            return full.to(dtype)

        dw1 = scatter(_fold_weight_grad(dw1e, g.Cb), (2, g.nb, g.Cb, g.Cb), dt[0])
        dw2 = scatter(_fold_weight_grad(dw2e, g.Cb), (2, g.nb, g.Cb, g.Cb), dt[2])
        db1 = scatter(torch.stack([db1e[:, :g.Cb], db1e[:, g.Cb:]]), (2, g.nb, g.Cb), dt[1])
        db2 = scatter(torch.stack([db2e[:, :g.Cb], db2e[:, g.Cb:]]), (2, g.nb, g.Cb), dt[3])
        return dx, dw1, db1, dw2, db2, None, None, None, None, (d if ctx.has_residual else None)


def _rows_c2r_local(lib, Y, out, addends, g, kweight, st):
    """Inverse row transform on one GPU; up to two ``[T, C]`` bf16 ``addends`` are summed into the stored tokens."""
    if addends:
        a0 = addends[0]
        a1 = addends[1] if len(addends) > 1 else None
        rc = lib.pnm_afno_rows_c2r_add(Y.data_ptr(), out.data_ptr(), a0.data_ptr(), None if a1 is None else a1.data_ptr(), g.arr,
                                       g.Tp, kweight, st)
        if rc == 0:
            return
        if rc != -2:
            _g._check(rc, "pnm_afno_rows_c2r_add")
    rc = lib.pnm_afno_rows_c2r(Y.data_ptr(), _ptrs8([out.data_ptr()]), g.arr, g.Tp, kweight, 0, None, 0, 1, 0, 0, None, None, st)
    _g._check(rc, "pnm_afno_rows_c2r")
    for a in addends:                       # shapes that take the fallback row kernel
        out.add_(a)


class _AfnoFilterFn(torch.autograd.Function):
    """tokens [Tp, C] bf16 (this rank's tokens, all channels) -> filtered tokens [Tp, C] bf16; block MLP in fp32 inside
    the column kernel (the path for fp32-exact filters)."""

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
                exchange: Optional[TokenChannelExchange] = None, mlp: str = "bf16", add_input: bool = False,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Filtered tokens: ``tokens`` is this rank's ``[Tp, C]`` bf16 slice of the token tensor.  ``add_input`` adds the
    tokens themselves (the layer's residual) and ``residual`` one more ``[Tp, C]`` bf16 tensor (the block's skip) to the
    result; on one GPU with the tensor-core MLP both sums happen in the store of the inverse row transform.

    ``mlp="bf16"`` runs the block MLP as tcgen05 GEMMs on the bf16 ``[real | imag]`` spectrum (what the reference's
    einsums do under bf16 autocast); ``mlp="fp32"`` keeps it in fp32 inside the column kernel."""
    fn = _AfnoFilterTcFn if (mlp == "bf16" and geo.Cb % 4 == 0) else _AfnoFilterFn
    if fn is _AfnoFilterTcFn and exchange is None and (add_input or residual is not None):
        if residual is not None and (residual.dtype != torch.bfloat16 or residual.shape != tokens.shape):
            raise ValueError("residual must be a bf16 tensor of the tokens' shape")
        return fn.apply(tokens, w1, b1, w2, b2, geo, float(sparsity_threshold), None, add_input, residual)
    out = fn.apply(tokens, w1, b1, w2, b2, geo, float(sparsity_threshold), exchange)
    if add_input:
        out = out + tokens
    return out if residual is None else out + residual
