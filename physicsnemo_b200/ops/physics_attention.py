"""Fused Transolver physics attention for irregular meshes (sm_100a).

Mathematics of ``physicsnemo/nn/module/physics_attention.py:501-558`` restated so that
every pass over the N points is a tcgen05 GEMM and everything else is four small kernels:

1. ``in_project_x`` followed by ``in_project_slice`` is one affine map (no nonlinearity in
   between): ``logits = xn @ Wc.T + bc`` with ``Wc = blockdiag_H(Ws) @ Wx``; the temperature
   division and the softmax over the S=64 slices of each head run in the GEMM epilogue, so
   neither ``x_mid`` nor the logits ever reach memory.  ``w`` (N, H*S) is the only large
   intermediate.
2. slice tokens ``Σ_n w[n,h,s] fx[n,h,:]`` and norms ``Σ_n w[n,h,s]`` come from one
   reduction GEMM ``w.T @ fx`` (+ column sums of ``w`` from an extra ones-column MMA); the
   per-head blocks are its diagonal blocks.  Under point sharding these partial sums are what
   crosses ranks: the GEMM writes them into a region of the rank's symmetric buffer, a flag is
   raised, and the token kernel of every rank adds the P copies with direct peer loads in its
   prologue — no stand-alone collective.
3. attention among the 64 tokens per head, the normalisation before it and the combined
   de-slicing matrix after it are one kernel (``pnm_pa_tokens_fwd``), one CTA per head.
4. de-slicing followed by ``out_linear`` is again one affine map:
   ``out = w @ Wcomb.T + bo (+ residual)`` with ``Wcomb = Wo @ blockdiag(out_tokens).T``.

The backward mirrors this: softmax Jacobian in GEMM epilogues, the token-sized backward
(attention, normalisation, ``dWo``, ``dWqkv`` and the operands of the point-sized GEMMs) in
``pnm_pa_tokens_bwd`` — which again sums the one quantity that crosses ranks (``dWcomb``) in its
prologue — and the gradients of ``Wx, bx, Ws, bs, T`` in ``pnm_pa_prepare_bwd``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import gemm as G
from . import pa_small as P


class LocalExchange:
    """Stand-in of ``parallel.peer.PeerRegions`` for an unsharded model: ordinary local buffers, no flags."""

    world = 1

    def region(self, floats: int, device) -> tuple:
        buf = torch.empty(floats, dtype=torch.float32, device=device)
        return buf, [buf.data_ptr()]

    def publish(self):
        return None


_LOCAL = LocalExchange()


class _PhysAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xn, res, H, D, S, exchange, Wx, bx, Wfx, bfx, Ws, bs, temp, Wqkv, Wo, bo):
        ex = exchange if exchange is not None else _LOCAL
        HS, inner = H * S, H * D
        dev = xn.device
        Wc, bc, inv_t, Wfx16, Wback = P.prepare_fwd(Wx.detach(), bx.detach(), Wfx.detach(), Ws.detach(), bs.detach(),
                                                    temp.detach().reshape(-1), H, D)
        fx = G.gemm_tn(xn, Wfx16, bias=bfx.detach().float())
        w = G.gemm_tn(xn, Wc, bias=bc, scale=inv_t, act=G.ACT_SOFTMAX64)
        # token sums [H*S, inner] followed by the slice norms [H*S]: partial sums of this rank's points
        buf, srcs = ex.region(HS * inner + HS, dev)
        buf.zero_()
        G.gemm_nt(w, fx, out=buf[: HS * inner].view(HS, inner), colsum_out=buf[HS * inner:])
        peer = ex.publish()
        Wcomb16, saved = P.tokens_fwd(srcs, HS * inner, inner, Wqkv.detach(), Wo.detach(), H, D, peer)
        out = G.gemm_tn(w, Wcomb16, bias=bo.detach().float(), aux=res, aux_mode=G.AUX_ADD if res is not None else G.AUX_NONE)
        ctx.save_for_backward(xn, fx, w, Wx, bx, Ws, temp, Wqkv, Wo, inv_t, Wback, *saved)
        ctx.dims = (H, D, S)
        ctx.exchange = ex
        ctx.has_res = res is not None
        ctx.param_dtypes = [t.dtype for t in (Wx, bx, Wfx, bfx, Ws, bs, temp, Wqkv, Wo, bo)]
        ctx.temp_shape = temp.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        xn, fx, w, Wx, bx, Ws, temp, Wqkv, Wo, inv_t, Wback, *saved = ctx.saved_tensors
        H, D, S = ctx.dims
        ex = ctx.exchange
        HS, inner = H * S, H * D
        Cout = Wo.shape[0]
        dout = dout.contiguous()
        dev = xn.device
        # out = w @ Wcomb.T + bo (+res): dWcomb [Cout, H*S] is a partial sum over this rank's points; dbo stays local
        buf, srcs = ex.region(Cout * HS, dev)
        buf.zero_()
        dbo = torch.zeros(Cout, dtype=torch.float32, device=dev)
        G.gemm_nt(dout, w, out=buf.view(Cout, HS), colsum_out=dbo)
        peer = ex.publish()
        # parameter gradients derived from the reduced dWcomb are global and equal on every rank; they are handed out as
        # 1/world shares so that the model-wide gradient sum over the shards restores them
        share = 1.0 / float(ex.world)
        dWo, dWqkv, d_norm, Bcat, BdT = P.tokens_bwd(srcs, Wqkv.detach(), Wo.detach(), saved, H, D, share, peer)
        # dw = [dout | fx] @ [Wcomb.T | blockdiag(d_tok)].T + d_norm ; softmax backward in the epilogue
        grp = torch.zeros(H, dtype=torch.float32, device=dev)
        dlogit = G.gemm_tn(dout, Bcat, a2=fx, bias=d_norm, aux=w, aux_mode=G.AUX_DSOFTMAX, scale=inv_t, scale_post=True,
                           group_out=grp)
        dfx = G.gemm_tn(w, BdT)                                                # d fx = w @ blockdiag(d_tok)
        dWc, dbc = G.gemm_nt(dlogit, xn, colsum=True)                         # (H*S, C), (H*S,)
        dWfx, dbfx = G.gemm_nt(dfx, xn, colsum=True)                          # (H*D, C), (H*D,)
        dWx, dbx, dWs, dbs, dtemp = P.prepare_bwd(dWc, dbc, grp, Wx.detach(), bx.detach(), Ws.detach(),
                                                  temp.detach().reshape(-1), H, D)
        dxn = G.gemm_tn(dlogit, Wback, a2=dfx)                                # [dlogit | dfx] @ [Wc ; Wfx]
        dres = dout if ctx.has_res else None
        grads = [dWx, dbx, dWfx, dbfx, dWs, dbs, dtemp.reshape(ctx.temp_shape), dWqkv, dWo, dbo]
        grads = [g if g.dtype == dt else g.to(dt) for g, dt in zip(grads, ctx.param_dtypes)]
        return (dxn, dres, None, None, None, None, *grads)


def fused_supported(mod) -> bool:
    """The kernels cover fp32 parameters, 64 slices and head widths that divide 256."""
    params = [mod.in_project_x.weight, mod.in_project_x.bias, mod.in_project_fx.weight, mod.in_project_fx.bias,
              mod.in_project_slice.weight, mod.in_project_slice.bias, mod.temperature, mod.qkv_project.weight,
              mod.out_linear.weight, mod.out_linear.bias]
    return P.supported(mod.heads, mod.dim_head, mod.slice_num, mod.in_project_x.weight.shape[1], params)


def physics_attention_irregular(mod, x: torch.Tensor, residual: torch.Tensor | None = None, exchange=None):
    """Fused forward of ``PhysicsAttentionIrregularMesh`` ``mod`` on ``x`` (B, N, C), B folded.

    ``exchange`` (optional, ``parallel.peer.PeerRegions``): where the partial sums that cross point shards live —
    once forward (slice tokens and norms) and once backward (the gradient of the combined de-slicing matrix, from
    which the token gradients follow).  All other parameter gradients stay per-shard partial sums.
    """
    B, N, C = x.shape
    outs = []
    for b in range(B):  # slice tokens are per sample; B is 1 in the point-cloud recipes
        # a view when B == 1: the backward of a select would zero-fill and copy the whole gradient
        xb = x.reshape(N, C) if B == 1 else x[b]
        if xb.dtype != torch.bfloat16:
            xb = xb.to(torch.bfloat16)
        rb = None
        if residual is not None:
            rb = residual.reshape(N, C) if B == 1 else residual[b]
            if rb.dtype != torch.bfloat16:
                rb = rb.to(torch.bfloat16)
            rb = rb.contiguous()
        out = _PhysAttnFn.apply(
            xb.contiguous(), rb, mod.heads, mod.dim_head, mod.slice_num, exchange,
            mod.in_project_x.weight, mod.in_project_x.bias, mod.in_project_fx.weight, mod.in_project_fx.bias,
            mod.in_project_slice.weight, mod.in_project_slice.bias, mod.temperature, mod.qkv_project.weight,
            mod.out_linear.weight, mod.out_linear.bias,
        )
        outs.append(out)
    return outs[0].unsqueeze(0) if B == 1 else torch.stack(outs)
