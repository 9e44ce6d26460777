"""AFNO on token shards: LayerNorm / MLP / patch embedding / head act on a rank's tokens, the spectral filter reshards
tokens ↔ channel blocks inside its Fourier kernels.

Reference: the channel-parallel ``DistributedAFNO`` (``physicsnemo/models/afno/distributed/afno.py:56-595``: channels split
over ``"model_parallel"``, an all-gather of activations and an fp32 all-reduce in every MLP) and the spatial
``DistributedRFFT2`` / ``DistributedIRFFT2`` (``physicsnemo/distributed/fft.py:66-244``: local FFT, ``all_to_all``
transpose, local FFT).  Here a rank owns ``tokens / P`` tokens everywhere except inside the filter, where it owns
``num_blocks / P`` channel blocks of ALL tokens; the two all-to-alls that this resharding implies are the load stage
of the forward row transform (peer loads) and the store stage of the inverse row transform (peer stores) —
``ops/afno_spectral.py``.  Parameters are replicated; their gradients are partial sums over the ranks (the filter
weights of a block are touched only by the block's owner).

``TokenShardedAFNO`` runs an unmodified ``AFNO`` module this way: same parameters, same state dict.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops import afno_spectral as A


def patch_tokens(x: torch.Tensor, patch: Tuple[int, int], channels_last_features: bool = False) -> torch.Tensor:
    """``[C, R*p0, W*p1]`` image rows → ``[R*W, C*p0*p1]`` patch tokens (feature order ``(c, p0, p1)``, the layout of a
    strided convolution's weight), or ``(p0, p1, c)`` with ``channels_last_features`` (the layout of the model's head)."""
    C, Hh, Ww = x.shape
    p0, p1 = patch
    t = x.reshape(C, Hh // p0, p0, Ww // p1, p1)
    t = t.permute(1, 3, 2, 4, 0) if channels_last_features else t.permute(1, 3, 0, 2, 4)
    return t.reshape((Hh // p0) * (Ww // p1), C * p0 * p1)


class TokenShardedAFNO:
    """Runs ``model`` (an ``AFNO``) on this rank's slice of the token sequence.

    ``forward(image_rows, first_token)``: ``image_rows`` = the pixel rows ``[C_in, R*p0, W]`` of ONE sample that cover
    this rank's tokens, ``first_token`` = offset of the rank's first token inside those rows.  Returns the head's
    output for the rank's tokens, ``[Tp, C_out * p0 * p1]`` with feature order ``(p0, p1, c)``.
    """

    def __init__(self, model, batch: int, group: Optional[dist.ProcessGroup] = None):
        self.model = model
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.h, self.w = model.h, model.w
        self.batch = batch
        T = batch * self.h * self.w
        nb = model.blocks[0].filter.num_blocks
        if T % self.world or nb % self.world:
            raise ValueError(f"{T} tokens and {nb} channel blocks must divide evenly over {self.world} ranks")
        self.Tp = T // self.world
        self.t0 = self.rank * self.Tp
        f = model.blocks[0].filter
        kept = int((self.h // 2 + 1) * f.hard_thresholding_fraction)
        self.geo = A.FilterGeometry(batch, self.h, self.w, model.embed_dim, nb, kept, self.rank, self.world)
        if not self.geo.supported() or f.hard_thresholding_fraction != 1 or f.hidden_size_factor != 1:
            raise ValueError("this AFNO configuration is outside what the fused spectral kernels cover")
        self.exchange = None
        dev = next(model.parameters()).device
        if self.world > 1 and dev.type == "cuda":
            self.exchange = A.TokenChannelExchange(group, self.Tp, model.embed_dim)
        per_img = self.h * self.w
        self.pos_index = (torch.arange(self.t0, self.t0 + self.Tp, device=dev) % per_img)

    def token_rows(self):
        """``(sample index, first patch row, last patch row + 1, offset of the first token in those rows)`` per sample
        that this rank's tokens touch (a list: a rank may span several samples when there are fewer ranks than samples)."""
        per_img = self.h * self.w
        out = []
        t, end = self.t0, self.t0 + self.Tp
        while t < end:
            b = t // per_img
            stop = min(end, (b + 1) * per_img)
            r0, r1 = (t % per_img) // self.w, ((stop - 1) % per_img) // self.w + 1
            out.append((b, r0, r1, (t % per_img) - r0 * self.w, stop - t))
            t = stop
        return out

    def forward(self, tokens_in: torch.Tensor) -> torch.Tensor:
        """``tokens_in``: ``[Tp, C_in * p0 * p1]`` patch tokens of this rank (feature order ``(c, p0, p1)``)."""
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=tokens_in.is_cuda):
            return self._forward(tokens_in)

    def _forward(self, tokens_in: torch.Tensor) -> torch.Tensor:
        m = self.model
        pe = m.patch_embed.proj
        x = ops.linear(tokens_in.to(torch.bfloat16), pe.weight.reshape(pe.weight.shape[0], -1), pe.bias)
        x = x + m.pos_embed[0, self.pos_index]          # fp32 like the stock forward: the first block's skip stays fp32
        for blk in m.blocks:
            f = blk.filter
            # bf16 tokens: each LayerNorm hands its input on as the skip tensor, so the two gradient paths of a skip are
            # summed inside the LayerNorm backward kernel instead of by a separate add (the first block's tokens are fp32)
            alias = x.dtype == torch.bfloat16
            if alias:
                xn, x = ops.layer_norm(x, blk.norm1.weight, blk.norm1.bias, blk.norm1.eps, return_residual=True)
            else:
                xn = ops.layer_norm(x, blk.norm1.weight, blk.norm1.bias, blk.norm1.eps)
            y = A.afno_filter(xn, f.w1, f.b1, f.w2, f.b2, self.geo, f.sparsity_threshold, self.exchange)
            x1 = y + xn                                             # the filter's own residual
            if blk.double_skip:
                x1 = x1 + x
                if x1.dtype == torch.bfloat16:
                    n2, res = ops.layer_norm(x1, blk.norm2.weight, blk.norm2.bias, blk.norm2.eps, return_residual=True)
                else:
                    n2, res = ops.layer_norm(x1, blk.norm2.weight, blk.norm2.bias, blk.norm2.eps), x1
            else:
                n2, res = ops.layer_norm(x1, blk.norm2.weight, blk.norm2.bias, blk.norm2.eps), x
            x = blk.mlp(n2, residual=res)
        return ops.linear(x, m.head.weight, None)

    __call__ = forward

    def step_done(self) -> None:
        if self.exchange is not None:
            self.exchange.step_done()
