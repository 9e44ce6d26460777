"""LayerNorm on the sm_100a kernels (``csrc/norm.cuh``) with a PyTorch oracle path.

Replaces ``torch.nn.LayerNorm`` / ``te.LayerNorm`` calls of the reference
(``physicsnemo/nn/module/layer_norm.py``, ``models/transolver/transolver.py:207-209``):
bf16 activations, fp32 statistics and parameters, optional fused residual add
(``y = LN(x + r)`` also returning ``x + r``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib
from . import gemm as _g


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, gamma, beta, eps, post=None, alias_out=False):
        lib = _lib.load(required=True)
        M, C = x2d.shape
        y = torch.empty_like(x2d)
        mean = torch.empty((M,), dtype=torch.float32, device=x2d.device)
        rstd = torch.empty((M,), dtype=torch.float32, device=x2d.device)
        g32 = gamma.detach().float().contiguous()
        b32 = beta.detach().float().contiguous() if beta is not None else None
        code = lib.pnm_layernorm_fwd(x2d.data_ptr(), None, g32.data_ptr(), None if b32 is None else b32.data_ptr(),
                                     y.data_ptr(), None, mean.data_ptr(), rstd.data_ptr(),
                                     None if post is None else post.data_ptr(), M, C, float(eps),
                                     _g._stream())
        _g._check(code, "pnm_layernorm_fwd")
        _g.launch_count += 1
        ctx.save_for_backward(x2d, g32, mean, rstd)
        ctx.has_beta = beta is not None
        ctx.has_post = post is not None
        ctx.param_dtype = gamma.dtype
        ctx.alias_out = alias_out
        if alias_out:
            return y, x2d.view_as(x2d)
        return y

    @staticmethod
    def backward(ctx, dy, dalias=None):
        lib = _lib.load(required=True)
        x2d, g32, mean, rstd = ctx.saved_tensors
        if dalias is not None:
            dalias = dalias.contiguous()
        M, C = x2d.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x2d)
        dgamma = torch.empty((C,), dtype=torch.float32, device=x2d.device)
        dbeta = torch.empty((C,), dtype=torch.float32, device=x2d.device)
        nfl = lib.pnm_layernorm_bwd_scratch_floats(M, C)
        scratch = torch.empty((nfl,), dtype=torch.float32, device=x2d.device)
        code = lib.pnm_layernorm_bwd(dy.data_ptr(), x2d.data_ptr(), g32.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                     None if dalias is None else dalias.data_ptr(), dx.data_ptr(), dgamma.data_ptr(),
                                     dbeta.data_ptr(), scratch.data_ptr(), M, C, _g._stream())
        _g._check(code, "pnm_layernorm_bwd")
        _g.launch_count += 2
        return (dx, dgamma.to(ctx.param_dtype), (dbeta.to(ctx.param_dtype) if ctx.has_beta else None), None,
                dy if ctx.has_post else None, None)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float = 1e-5,
               post: Optional[torch.Tensor] = None, return_residual: bool = False):
    """LayerNorm over the last dimension; ``post`` (same shape) is added to the result.

    ``return_residual=True`` returns ``(LN(x), x')`` where ``x'`` is ``x`` itself, routed through the
    same autograd node: a pre-norm residual block that consumes ``x'`` as its skip connection gets the
    sum of the two gradient paths from the LayerNorm backward kernel instead of a separate add.
    """
    C = x.shape[-1]
    if not _g.fused_path_enabled(x) or C % 8 or C > 1024:
        y = F.layer_norm(x, (C,), weight, bias, eps)
        y = y if post is None else y + post
        return (y, x) if return_residual else y
    x2 = x.reshape(-1, C)
    if x2.dtype != torch.bfloat16:
        x2 = x2.to(torch.bfloat16)
    x2 = x2.contiguous()
    p2 = None
    if post is not None:
        p2 = post.reshape(-1, C)
        if p2.dtype != torch.bfloat16:
            p2 = p2.to(torch.bfloat16)
        p2 = p2.contiguous()
    if return_residual:
        y, alias = _LayerNormFn.apply(x2, weight, bias, eps, p2, True)
        return y.reshape(x.shape), alias.reshape(x.shape)
    return _LayerNormFn.apply(x2, weight, bias, eps, p2).reshape(x.shape)
