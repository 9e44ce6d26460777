"""EDM noise conditioning in one launch (``pnm_edm_conditioning`` in ``csrc/elementwise.cu``).

``edm_conditioning(noise, freqs, w0, b0, w1, b1, extra=None)`` returns
``silu(W1 silu(W0 ([sin(noise f), cos(noise f)] + extra) + b0) + b1)`` as fp32 ``[B, E]``: the positional embedding with
swapped halves, the optional class / augmentation term and the two ``Linear + SiLU`` layers of the diffusion U-Nets
(``SongUNet.conditioning_embedding``), which are five small launches otherwise.  The backward recomputes the chain with
tensor operations (it is a few kFLOP), so the op is differentiable in the weights, biases and ``extra``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from . import gemm as _g


def _lib_cond():
    lib = _lib.load(required=True)
    if not getattr(lib, "_cond_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.pnm_edm_conditioning.argtypes = [vp] * 8 + [i, i, i, i, vp]
        lib.pnm_edm_conditioning.restype = i
        lib._cond_declared = True
    return lib


def reference(noise, freqs, w0, b0, w1, b1, extra=None):
    ang = noise.float().ger(freqs.float())
    emb = torch.cat([ang.sin(), ang.cos()], dim=1)
    if extra is not None:
        emb = emb + extra.float()
    h = F.silu(F.linear(emb, w0.float(), b0.float() if b0 is not None else None))
    return F.silu(F.linear(h, w1.float(), b1.float() if b1 is not None else None))


def supported(noise, freqs, w0, w1) -> bool:
    C, E = w0.shape[1], w0.shape[0]
    return (noise.is_cuda and w0.dtype in (torch.float32, torch.bfloat16) and w1.dtype == w0.dtype and freqs.numel() * 2 == C
            and w1.shape == (E, E) and (C + E) * 4 <= 48 * 1024 and noise.dim() == 1)


class _EDMConditioning(torch.autograd.Function):
    @staticmethod
    def forward(ctx, noise, freqs, w0, b0, w1, b1, extra):
        B, (E, C) = noise.shape[0], w0.shape
        out = torch.empty(B, E, dtype=torch.float32, device=noise.device)
        cast = lambda t: None if t is None else t.detach().to(w0.dtype).contiguous()  # noqa: E731
        n32, f32 = noise.detach().float().contiguous(), freqs.detach().float().contiguous()
        x32 = None if extra is None else extra.detach().float().contiguous()
        w0c, w1c, b0c, b1c = w0.detach().contiguous(), w1.detach().contiguous(), cast(b0), cast(b1)
        ptr = lambda t: None if t is None else t.data_ptr()  # noqa: E731
        err = _lib_cond().pnm_edm_conditioning(n32.data_ptr(), f32.data_ptr(), ptr(x32), w0c.data_ptr(), ptr(b0c), w1c.data_ptr(), ptr(b1c),
                                               out.data_ptr(), B, C, E, 1 if w0.dtype == torch.float32 else 0,
                                               torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_edm_conditioning failed ({err})")
        _g.launch_count += 1
        ctx.save_for_backward(noise, freqs, w0, b0, w1, b1, extra)
        return out

    @staticmethod
    def backward(ctx, grad):
        saved = ctx.saved_tensors
        noise, freqs = saved[0], saved[1]
        with torch.enable_grad():
            leaves = [None if t is None else t.detach().requires_grad_(t.requires_grad) for t in saved[2:]]
            w0, b0, w1, b1, extra = leaves
            out = reference(noise, freqs, w0, b0, w1, b1, extra)
            wanted = [t for t in leaves if t is not None and t.requires_grad]
            grads = iter(torch.autograd.grad(out, wanted, grad) if wanted else ())
        return (None, None, *[next(grads) if (t is not None and t.requires_grad) else None for t in leaves])


def edm_conditioning(noise, freqs, w0, b0, w1, b1, extra=None):
    if supported(noise, freqs, w0, w1):
        return _EDMConditioning.apply(noise, freqs, w0, b0, w1, b1, extra)
    return reference(noise, freqs, w0, b0, w1, b1, extra)
