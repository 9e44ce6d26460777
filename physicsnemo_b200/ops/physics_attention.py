"""Fused Transolver physics attention for irregular meshes (sm_100a).

Mathematics of ``physicsnemo/nn/module/physics_attention.py:501-558`` restated so that
every pass over the N points is a tcgen05 GEMM:

1. ``in_project_x`` followed by ``in_project_slice`` is one affine map (no nonlinearity in
   between): ``logits = xn @ Wc.T + bc`` with ``Wc = blockdiag_H(Ws) @ Wx``; the temperature
   division and the softmax over the S=64 slices of each head run in the GEMM epilogue, so
   neither ``x_mid`` nor the logits ever reach memory.  ``w`` (N, H*S) is the only large
   intermediate.
2. slice tokens ``Σ_n w[n,h,s] fx[n,h,:]`` and norms ``Σ_n w[n,h,s]`` come from one
   reduction GEMM ``w.T @ fx`` (+ column sums of ``w`` from an extra ones-column MMA); the
   per-head blocks are its diagonal blocks.  Under point sharding these H*S*(D+1) partial
   sums are what crosses ranks (one all-reduce).
3. attention among the 64 tokens per head is tiny and stays in PyTorch (fp32, autograd).
4. de-slicing followed by ``out_linear`` is again one affine map:
   ``out = w @ Wcomb.T + bo (+ residual)`` with ``Wcomb = Wo @ blockdiag(out_tokens).T``.

The backward mirrors this with the softmax Jacobian, GELU-free, in GEMM epilogues; the
small matrices (``Wc``, ``Wcomb``, tokens) are differentiated by autograd on a side graph.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import gemm as G


def _blockdiag(blocks: torch.Tensor) -> torch.Tensor:
    """(H, a, b) -> (H*a, H*b) block-diagonal matrix (differentiable)."""
    return torch.block_diag(*blocks.unbind(0))


def _diag_blocks(m: torch.Tensor, H: int) -> torch.Tensor:
    """(H*a, H*b) -> (H, a, b): the diagonal blocks."""
    a, b = m.shape[0] // H, m.shape[1] // H
    return torch.stack([m[h * a:(h + 1) * a, h * b:(h + 1) * b] for h in range(H)])


class _PhysAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xn, res, H, D, S, reduce_fn, Wx, bx, Wfx, bfx, Ws, bs, temp, Wqkv, Wo, bo):
        M = xn.shape[0]
        params = [Wx, bx, Wfx, bfx, Ws, bs, temp, Wqkv, Wo, bo]
        with torch.enable_grad():
            p = [t.detach().float().requires_grad_(True) for t in params]
            pWx, pbx, pWfx, pbfx, pWs, pbs, ptemp, pWqkv, pWo, pbo = p
            bd_ws = _blockdiag(pWs.unsqueeze(0).expand(H, S, D))            # (H*S, H*D)
            Wc = bd_ws @ pWx                                                  # (H*S, C)
            bc = bd_ws @ pbx + pbs.repeat(H)                                  # (H*S,)
            inv_t = (1.0 / torch.clamp(ptemp.reshape(H), min=0.5, max=5.0)).repeat_interleave(S)
        fx = G.gemm_tn(xn, G._bf16_weight(Wfx), bias=pbfx.detach())
        w = G.gemm_tn(xn, Wc.detach().to(torch.bfloat16), bias=bc.detach(), scale=inv_t.detach().contiguous(),
                      act=G.ACT_SOFTMAX64)
        tok_full, norm_full = G.gemm_nt(w, fx, colsum=True)                   # (H*S, H*D) fp32, (H*S,)
        tok_raw = _diag_blocks(tok_full, H)                                    # (H, S, D)
        norm_raw = norm_full.reshape(H, S)
        if reduce_fn is not None:  # point-sharded: partial sums -> global sums
            packed = torch.cat([tok_raw.reshape(-1), norm_raw.reshape(-1)])
            packed = reduce_fn(packed)
            tok_raw = packed[: H * S * D].reshape(H, S, D)
            norm_raw = packed[H * S * D:].reshape(H, S)
        with torch.enable_grad():
            tok_leaf = tok_raw.detach().requires_grad_(True)
            norm_leaf = norm_raw.detach().requires_grad_(True)
            token = tok_leaf / (norm_leaf + 1e-2).unsqueeze(-1)              # (H, S, D)
            qkv = token @ pWqkv.t()                                           # (H, S, 3D)
            q, k, v = qkv.reshape(H, S, 3, D).unbind(2)
            out_tok = F.scaled_dot_product_attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)).squeeze(0)
            Wcomb = pWo @ _blockdiag(out_tok).t()                             # (C, H*D) @ (H*D, H*S) -> (C, H*S)
        out = G.gemm_tn(w, Wcomb.detach().to(torch.bfloat16), bias=pbo.detach(), aux=res,
                        aux_mode=G.AUX_ADD if res is not None else G.AUX_NONE)
        ctx.save_for_backward(xn, fx, w)
        ctx.graph = (p, Wc, bc, inv_t, tok_leaf, norm_leaf, Wcomb)
        ctx.dims = (H, D, S)
        ctx.reduce_fn = reduce_fn
        ctx.has_res = res is not None
        ctx.param_dtypes = [t.dtype for t in params]
        return out

    @staticmethod
    def backward(ctx, dout):
        xn, fx, w = ctx.saved_tensors
        p, Wc, bc, inv_t, tok_leaf, norm_leaf, Wcomb = ctx.graph
        H, D, S = ctx.dims
        dout = dout.contiguous()
        dev = xn.device
        # out = w @ Wcomb.T + bo (+res)
        dWcomb, dbo = G.gemm_nt(dout, w, colsum=True)                         # (C, H*S), (C,)
        share = 1.0
        if ctx.reduce_fn is not None:
            # the slice tokens are global quantities: their gradient needs the global dWcomb.
            packed = ctx.reduce_fn(torch.cat([dWcomb.reshape(-1), dbo]))
            dWcomb, dbo = packed[: dWcomb.numel()].reshape(dWcomb.shape), packed[dWcomb.numel():]
            # parameter gradients derived from reduced quantities are already global and equal on
            # every rank; they are handed out as 1/world shares so that the model-wide gradient
            # sum over the shards restores them.
            share = 1.0 / float(getattr(ctx.reduce_fn, "world", None) or getattr(getattr(ctx.reduce_fn, "__self__", None), "world", 1))
        pWo, pWqkv = p[8], p[7]
        d_tok, d_norm, dWo, dWqkv = torch.autograd.grad(Wcomb, [tok_leaf, norm_leaf, pWo, pWqkv], dWcomb,
                                                         retain_graph=False)
        # dw = [dout | fx] @ [Wcomb.T | blockdiag(d_tok)].T + d_norm ; softmax backward in the epilogue
        bd_dtok = _blockdiag(d_tok)                                           # (H*S, H*D)
        Bcat = torch.cat([Wcomb.detach().t(), bd_dtok], dim=1).to(torch.bfloat16).contiguous()  # (H*S, C + H*D)
        grp = torch.zeros(H, dtype=torch.float32, device=dev)
        dlogit = G.gemm_tn(dout, Bcat, a2=fx, bias=d_norm.reshape(-1).contiguous(), aux=w, aux_mode=G.AUX_DSOFTMAX,
                           scale=inv_t.detach().contiguous(), scale_post=True, group_out=grp)
        # d fx = w @ blockdiag(d_tok)
        dfx = G.gemm_tn(w, bd_dtok.t().to(torch.bfloat16).contiguous())
        dWc, dbc = G.gemm_nt(dlogit, xn, colsum=True)                         # (H*S, C), (H*S,)
        dWfx, dbfx = G.gemm_nt(dfx, xn, colsum=True)                          # (H*D, C), (H*D,)
        d_inv_t = (grp / inv_t.detach().reshape(H, S)[:, 0]).repeat_interleave(S) / S
        pWx, pbx, pWs, pbs, ptemp = p[0], p[1], p[4], p[5], p[6]
        dWx, dbx, dWs, dbs, dtemp = torch.autograd.grad([Wc, bc, inv_t], [pWx, pbx, pWs, pbs, ptemp],
                                                        [dWc, dbc, d_inv_t], allow_unused=True)
        # d xn = [dlogit | dfx] @ [Wc ; Wfx]
        Wback = torch.cat([Wc.detach().t(), p[2].detach().t()], dim=1).to(torch.bfloat16).contiguous()  # (C, H*S + H*D)
        dxn = G.gemm_tn(dlogit, Wback, a2=dfx)
        dres = dout if ctx.has_res else None
        if share != 1.0:
            dWqkv, dWo, dbo = dWqkv * share, dWo * share, dbo * share
        grads = [dWx, dbx, dWfx, dbfx, dWs, dbs, dtemp, dWqkv, dWo, dbo]
        grads = [None if g is None else g.to(dt) for g, dt in zip(grads, ctx.param_dtypes)]
        ctx.graph = None
        return (dxn, dres, None, None, None, None, *grads)


def physics_attention_irregular(mod, x: torch.Tensor, residual: torch.Tensor | None = None, reduce_fn=None):
    """Fused forward of ``PhysicsAttentionIrregularMesh`` ``mod`` on ``x`` (B, N, C), B folded.

    ``reduce_fn`` (optional) maps a flat fp32 tensor of partial sums to the sum over all point
    shards (an all-reduce); it is applied once forward (slice tokens and norms) and once
    backward (the gradient of the combined de-slicing matrix, from which the token gradients
    follow).  All other parameter gradients stay per-shard partial sums.
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
            xb.contiguous(), rb, mod.heads, mod.dim_head, mod.slice_num, reduce_fn,
            mod.in_project_x.weight, mod.in_project_x.bias, mod.in_project_fx.weight, mod.in_project_fx.bias,
            mod.in_project_slice.weight, mod.in_project_slice.bias, mod.temperature, mod.qkv_project.weight,
            mod.out_linear.weight, mod.out_linear.bias,
        )
        outs.append(out)
    return outs[0].unsqueeze(0) if B == 1 else torch.stack(outs)
