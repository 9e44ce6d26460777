"""Pixel / observation cross attention with fused key / value projections, and the counting sort that packs
observations by pixel (``csrc/pixel_attn.cu``).

Every grid pixel ``p`` attends over its own list of observation tokens ``tokens[cu[p]:cu[p+1]]`` (grouped-query
attention: ``n_q_heads`` query heads share ``n_kv_heads`` key / value heads).  The reference fuses the per-token
projections ``K = tok W_k^T``, ``V = tok W_v^T + b`` into a Triton attention kernel
(``physicsnemo/experimental/models/healda/kernels/pixel_attention.py:221-1425``).  Here the projections are re-associated
onto the pixel side instead::

    scores[t, h] = tok_t . (W_k[kv(h)]^T q_h) * scale          ->  qk = (scale * Q) W_k          (dense GEMM)
    out[h]       = (sum_t w[t, h] tok_t) W_v[kv(h)]^T + b      ->  out = ctx W_v^T + b           (dense GEMM)

so no key or value is ever formed per token, and the variable-length part is one kernel that reads every token once per
block of 16 heads and works in the token dimension (``ctx = softmax(tok qk^T) tok``).  Its backward kernel recomputes
the probabilities from the saved log-sum-exp; the GEMMs differentiate through autograd.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from . import gemm as _g

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _lib_pa():
    lib = _lib.load(required=True)
    if not getattr(lib, "_pa_declared", False):
        vp, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.pnm_pixel_attn_fwd.argtypes = [vp] * 5 + [i, i, i, i, vp]
        lib.pnm_pixel_attn_bwd.argtypes = [vp] * 8 + [i, i, i, i64, i, i, vp]
        lib.pnm_counting_histogram.argtypes = [vp, vp, i64, i, vp, vp]
        lib.pnm_counting_scatter.argtypes = [vp, vp, vp, vp, i64, i, vp]
        for f in (lib.pnm_pixel_attn_fwd, lib.pnm_pixel_attn_bwd, lib.pnm_counting_histogram, lib.pnm_counting_scatter):
            f.restype = i
        lib._pa_declared = True
    return lib


# ------------------------------------------------------------------------------------------------ token attention
def token_attention_reference(qk: torch.Tensor, tokens: torch.Tensor, cu_seqlens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``ctx[p, h] = softmax_t(tokens_p qk[p, h]) tokens_p`` with dense padding (any device); returns ``(ctx, lse)``."""
    P, H, Dt = qk.shape
    cu = cu_seqlens.long()
    n = cu[1:] - cu[:-1]
    nmax = int(n.max()) if P else 0
    if nmax == 0:
        return qk * 0.0, qk.new_full((P, H), float("-inf"), dtype=torch.float32)
    slot = torch.arange(nmax, device=qk.device)[None, :]
    valid = slot < n[:, None]                                                    # [P, nmax]
    gather = (cu[:-1, None] + slot).clamp(max=max(tokens.shape[0] - 1, 0))
    cd = torch.float64 if qk.dtype == torch.float64 else torch.float32
    tok = tokens.to(cd)[gather] * valid[..., None]                                # [P, nmax, Dt]
    s = torch.einsum("pnc,phc->phn", tok, qk.to(cd)).masked_fill(~valid[:, None, :], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    w = torch.exp(s - lse.masked_fill(lse == float("-inf"), 0.0)[..., None]).masked_fill(~valid[:, None, :], 0.0)
    return torch.einsum("phn,pnc->phc", w, tok).to(qk.dtype), lse


def token_attention_supported(qk: torch.Tensor, tokens: torch.Tensor) -> bool:
    return (qk.is_cuda and qk.dtype in _DT and tokens.dtype == qk.dtype and qk.shape[-1] in (32, 64, 96, 128)
            and qk.shape[0] > 0 and tokens.shape[0] > 0)


class _TokenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qk, tokens, cu):
        P, H, Dt = qk.shape
        qk, tokens = qk.contiguous(), tokens.contiguous()
        cu32 = cu.to(torch.int32).contiguous()
        out = torch.empty_like(qk)
        lse = torch.empty(P, H, dtype=torch.float32, device=qk.device)
        err = _lib_pa().pnm_pixel_attn_fwd(qk.data_ptr(), tokens.data_ptr(), cu32.data_ptr(), out.data_ptr(), lse.data_ptr(), P, H, Dt,
                                           _DT[qk.dtype], torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_pixel_attn_fwd failed ({err})")
        _g.launch_count += 1
        ctx.save_for_backward(qk, tokens, cu32, out, lse)
        return out

    @staticmethod
    def backward(ctx, dout):
        qk, tokens, cu32, out, lse = ctx.saved_tensors
        P, H, Dt = qk.shape
        dout = dout.contiguous().to(qk.dtype)
        delta = (dout.float() * out.float()).sum(-1).contiguous()
        dqk = torch.empty(P, H, Dt, dtype=torch.float32, device=qk.device)
        N, blocks = tokens.shape[0], (H + 15) // 16
        # every block of 16 heads writes its own slab of token gradients (summed below) unless the slabs would be large
        atomic = blocks > 1 and blocks * N * Dt * 4 > (2 << 30)
        dtok = (torch.zeros(N, Dt, dtype=torch.float32, device=qk.device) if atomic
                else torch.empty(blocks, N, Dt, dtype=torch.float32, device=qk.device))
        err = _lib_pa().pnm_pixel_attn_bwd(qk.data_ptr(), tokens.data_ptr(), cu32.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                           delta.data_ptr(), dqk.data_ptr(), dtok.data_ptr(), P, H, Dt, N, int(atomic), _DT[qk.dtype],
                                           torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_pixel_attn_bwd failed ({err})")
        _g.launch_count += 1
        empty = (cu32[1:] == cu32[:-1])[:, None, None]
        if not atomic:
            # rows cu[P]..N (tokens that belong to no pixel) are never written: mask them
            dtok = dtok[0] if blocks == 1 else dtok.sum(0)
            if int(cu32[-1]) < N:
                dtok[int(cu32[-1]):] = 0
        return dqk.masked_fill(empty, 0.0).to(qk.dtype), dtok.to(tokens.dtype), None


def token_attention(qk: torch.Tensor, tokens: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    if token_attention_supported(qk, tokens):
        return _TokenAttention.apply(qk, tokens, cu_seqlens)
    return token_attention_reference(qk, tokens, cu_seqlens)[0]


# ------------------------------------------------------------------------------------------------ public operator
def pixel_attention(Q: torch.Tensor, tokens: torch.Tensor, W_k: torch.Tensor, W_v: torch.Tensor, cu_seqlens_k: torch.Tensor,
                    max_seqlen_k: int = 0, *, n_kv_heads: int, scale: float, B_k: Optional[torch.Tensor] = None,
                    B_v: Optional[torch.Tensor] = None, group_map=None) -> torch.Tensor:
    """Grouped-query cross attention of ``Q`` ``[P, n_q_heads, d_head]`` over packed ``tokens`` ``[N, token_dim]``.

    ``W_k`` / ``W_v`` are ``[n_kv_heads * d_head, token_dim]``.  A key bias shifts all scores of a head equally and
    cancels in the softmax, so ``B_k`` is accepted and ignored; ``B_v`` is added for pixels with at least one token.
    Pixels without tokens return zeros.  ``max_seqlen_k`` and ``group_map`` are scheduling hints of the reference
    kernel and are not needed here.
    """
    P, Hq, dh = Q.shape
    Dt = tokens.shape[1]
    if Hq % n_kv_heads:
        raise ValueError(f"n_q_heads={Hq} must be divisible by n_kv_heads={n_kv_heads}")
    g = Hq // n_kv_heads
    dt = Q.dtype
    qk = torch.einsum("pkgd,kdc->pkgc", (Q * scale).view(P, n_kv_heads, g, dh), W_k.to(dt).view(n_kv_heads, dh, Dt)).reshape(P, Hq, Dt)
    ctx = token_attention(qk, tokens.to(dt), cu_seqlens_k)
    out = torch.einsum("pkgc,kdc->pkgd", ctx.view(P, n_kv_heads, g, Dt), W_v.to(dt).view(n_kv_heads, dh, Dt)).reshape(P, Hq, dh)
    if B_v is not None:
        nonempty = (cu_seqlens_k[1:] != cu_seqlens_k[:-1]).to(dt)[:, None, None]
        out = out + nonempty * B_v.to(dt).view(n_kv_heads, 1, dh).expand(n_kv_heads, g, dh).reshape(1, Hq, dh)
    return out


# ------------------------------------------------------------------------------------------------- counting sort
def counting_sort_and_pack(flat_idx: torch.Tensor, total_pixels: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(order, counts)``: ``flat_idx[order]`` is non-decreasing and ``counts[b]`` is the number of entries equal to ``b``.

    On a GPU: histogram with atomics, exclusive scan, scatter with per-bin cursors (the order inside a bin is
    arbitrary; attention over a pixel's tokens does not depend on it).  Elsewhere: ``bincount`` + ``argsort``.
    """
    n = flat_idx.shape[0]
    if not flat_idx.is_cuda or n == 0:
        counts = torch.bincount(flat_idx.long(), minlength=total_pixels)
        return flat_idx.argsort(stable=True).int(), counts
    lib = _lib_pa()
    idx = flat_idx.to(torch.int32).contiguous()
    scratch = torch.zeros(2 * total_pixels + 1, dtype=torch.int32, device=idx.device)
    counts, cursor, bad = scratch[:total_pixels], scratch[total_pixels:2 * total_pixels], scratch[2 * total_pixels:]
    st = torch.cuda.current_stream().cuda_stream
    err = lib.pnm_counting_histogram(idx.data_ptr(), counts.data_ptr(), n, total_pixels, bad.data_ptr(), st)
    if err:
        raise RuntimeError(f"pnm_counting_histogram failed ({err})")
    offsets = (torch.cumsum(counts, 0, dtype=torch.int32) - counts).contiguous()
    order = torch.empty(n, dtype=torch.int32, device=idx.device)
    err = lib.pnm_counting_scatter(idx.data_ptr(), offsets.data_ptr(), cursor.data_ptr(), order.data_ptr(), n, total_pixels, st)
    if err:
        raise RuntimeError(f"pnm_counting_scatter failed ({err})")
    _g.launch_count += 2
    if int(bad):
        raise ValueError(f"flat_idx has entries outside [0, {total_pixels})")
    return order, counts.long()
