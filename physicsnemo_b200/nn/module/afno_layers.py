"""Adaptive Fourier Neural Operator layers.

Parity: ``physicsnemo/nn/module/afno_layers.py`` — ``AFNOMlp`` (``:37``), ``AFNO2DLayer``
(``:99-327``: fp32 ``rfft2(ortho)`` over (H, W) of a BHWC tensor, block-diagonal complex two-layer
MLP with ReLU on the retained modes, soft-shrink, ``irfft2``, residual; parameters
``w1[2,nb,bs,bs*f]``, ``b1``, ``w2``, ``b2``), ``AFNOPatchEmbed`` (``:330-411``), ``ScaleShiftMlp``,
``ModAFNOMlp``, ``ModAFNO2DLayer`` (modulated variants).

The spectral MLP is evaluated on the retained window only and written once into a zero
spectrum; ``AFNOMlp`` (and LayerNorm in the blocks) take the fused sm_100a kernels on CUDA
bf16 inputs.
"""
from __future__ import annotations

from typing import List, Tuple, Union

import torch
import torch.fft as fft
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ... import ops
from .activations import activation_code


class AFNOMlp(nn.Module):
    """``fc2(drop(act(fc1(x))))`` followed by dropout."""

    def __init__(self, in_features: int, latent_features: int, out_features: int,
                 activation_fn: nn.Module = nn.GELU(), drop: float = 0.0):
        super().__init__()
        self.fc1 = nn.Linear(in_features, latent_features)
        self.act = activation_fn
        self.fc2 = nn.Linear(latent_features, out_features)
        self.drop = nn.Dropout(drop)

    def forward(self, x: Tensor, residual: Tensor | None = None) -> Tensor:
        code = activation_code(self.act)
        if code is not None and (self.drop.p == 0.0 or not self.training) and ops.fused_path_enabled(x):
            return ops.mlp_chain(x, [self.fc1.weight, self.fc2.weight], [self.fc1.bias, self.fc2.bias], [code, 0],
                                 residual=residual)
        x = self.drop(self.act(self.fc1(x)))
        x = self.drop(self.fc2(x))
        return x if residual is None else x + residual


def _block_cmul(xr, xi, w, b):
    """(xr + i xi) @ (w[0] + i w[1]) + (b[0] + i b[1]) per block; returns (real, imag)."""
    e = lambda a, m: torch.einsum("nyxbi,bio->nyxbo", a, m)  # noqa: E731
    return e(xr, w[0]) - e(xi, w[1]) + b[0], e(xi, w[0]) + e(xr, w[1]) + b[1]


class AFNO2DLayer(nn.Module):
    """Spectral token mixer of AFNO; input / output (B, H, W, C)."""

    def __init__(self, hidden_size: int, num_blocks: int = 8, sparsity_threshold: float = 0.01,
                 hard_thresholding_fraction: float = 1, hidden_size_factor: int = 1):
        super().__init__()
        if hidden_size % num_blocks != 0:
            raise ValueError(f"hidden_size {hidden_size} should be divisible by num_blocks {num_blocks}")
        self.hidden_size, self.num_blocks = hidden_size, num_blocks
        self.sparsity_threshold = sparsity_threshold
        self.block_size = hidden_size // num_blocks
        self.hard_thresholding_fraction, self.hidden_size_factor = hard_thresholding_fraction, hidden_size_factor
        self.scale = 0.02
        bs, f = self.block_size, hidden_size_factor
        self.w1 = nn.Parameter(self.scale * torch.randn(2, num_blocks, bs, bs * f))
        self.b1 = nn.Parameter(self.scale * torch.randn(2, num_blocks, bs * f))
        self.w2 = nn.Parameter(self.scale * torch.randn(2, num_blocks, bs * f, bs))
        self.b2 = nn.Parameter(self.scale * torch.randn(2, num_blocks, bs))

    def _spectral_mlp(self, xr, xi):
        o1r, o1i = _block_cmul(xr, xi, self.w1, self.b1)
        o1r, o1i = F.relu(o1r), F.relu(o1i)
        return _block_cmul(o1r, o1i, self.w2, self.b2)

    def forward(self, x: Tensor, residual: Tensor | None = None) -> Tensor:
        """``filter(x) + x`` (``+ residual`` when given: the skip connection of the surrounding block)."""
        if not torch.compiler.is_compiling():
            if x.ndim != 4:
                raise ValueError(f"Expected 4D input (B, H, W, C), got {x.ndim}D tensor with shape {tuple(x.shape)}")
        if residual is not None and not (type(x) is torch.Tensor and x.is_cuda and x.dtype == torch.bfloat16
                                         and residual.dtype == torch.bfloat16 and residual.shape == x.shape):
            return self.forward(x) + residual
        bias = x
        dtype = x.dtype
        B, H, W, C = x.shape
        if type(x) is torch.Tensor and ops.fused_path_enabled(x) and self.hard_thresholding_fraction == 1 \
                and self.hidden_size_factor == 1 and self.w1.dtype == torch.float32:
            # CUDA, bf16 compute: the library's own Fourier kernels (pruned row DFTs, two-level column DFT, complex block
            # MLP and soft-shrink in one kernel); no library FFT, no complex einsums
            from ...ops import afno_spectral as _af

            geo = _af.FilterGeometry(B, H, W, C, self.num_blocks, H // 2 + 1)
            if geo.supported():
                if dtype == torch.bfloat16:
                    # the layer's residual (and the block's skip) are added in the store of the inverse transform
                    y = _af.afno_filter(x.reshape(-1, C), self.w1, self.b1, self.w2, self.b2, geo, self.sparsity_threshold,
                                        add_input=True, residual=None if residual is None else residual.reshape(-1, C))
                    return y.reshape(B, H, W, C)
                y = _af.afno_filter(x.reshape(-1, C).to(torch.bfloat16), self.w1, self.b1, self.w2, self.b2, geo,
                                    self.sparsity_threshold)
                return y.reshape(B, H, W, C).to(dtype) + bias
        if residual is not None:
            return self.forward(x) + residual
        x = x.float()
        xf = fft.rfft2(x, dim=(1, 2), norm="ortho")
        Wf = W // 2 + 1
        total_modes = H // 2 + 1
        kept = int(total_modes * self.hard_thresholding_fraction)
        lo, hi = total_modes - kept, total_modes + kept
        win = xf[:, lo:hi, :kept].reshape(B, -1, min(kept, Wf), self.num_blocks, self.block_size)
        o2r, o2i = self._spectral_mlp(win.real, win.imag)
        o2 = torch.stack([o2r, o2i], dim=-1)
        o2 = F.softshrink(o2, lambd=self.sparsity_threshold)
        rows = win.shape[1]
        # zero spectrum with the window filled in (softshrink(0) = 0 outside the window)
        o2 = F.pad(o2, (0, 0, 0, 0, 0, 0, 0, Wf - win.shape[2], lo, H - lo - rows))
        xc = torch.view_as_complex(o2.contiguous()).reshape(B, H, Wf, C)
        x = fft.irfft2(xc, s=(H, W), dim=(1, 2), norm="ortho")
        return x.type(dtype) + bias


class AFNOPatchEmbed(nn.Module):
    """Non-overlapping patch embedding: (B, C, H, W) → (B, N, D) through a strided convolution."""

    def __init__(self, inp_shape: List[int], in_channels: int, patch_size: List[int] = [16, 16], embed_dim: int = 256):
        super().__init__()
        if len(inp_shape) != 2:
            raise ValueError("inp_shape should be a list of length 2")
        if len(patch_size) != 2:
            raise ValueError("patch_size should be a list of length 2")
        self.inp_shape, self.patch_size = inp_shape, patch_size
        self.num_patches = (inp_shape[1] // patch_size[1]) * (inp_shape[0] // patch_size[0])
        self.proj = nn.Conv2d(in_channels, embed_dim, kernel_size=patch_size, stride=patch_size)

    def forward(self, x: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            c, h, w = self.proj.in_channels, self.inp_shape[0], self.inp_shape[1]
            if x.ndim != 4 or x.shape[1] != c or x.shape[2] != h or x.shape[3] != w:
                raise ValueError(f"Expected input shape (B, {c}, {h}, {w}), got {tuple(x.shape)}")
        if type(x) is torch.Tensor and ops.fused_path_enabled(x):
            # stride == kernel: the convolution is a GEMM over non-overlapping patches
            B, C, H, W = x.shape
            p0, p1 = self.patch_size
            # one pass: the cast to bf16 writes the patch-major layout directly
            t = x.reshape(B, C, H // p0, p0, W // p1, p1).permute(0, 2, 4, 1, 3, 5)
            t = t.to(torch.bfloat16, memory_format=torch.contiguous_format).reshape(B, -1, C * p0 * p1)
            return ops.linear(t, self.proj.weight.reshape(self.proj.weight.shape[0], -1), self.proj.bias)
        return self.proj(x).flatten(2).transpose(1, 2)


class ScaleShiftMlp(nn.Module):
    """MLP producing ``(1 + scale, shift)`` modulation pairs from an embedding."""

    def __init__(self, in_features: int, out_features: int, hidden_features: Union[int, None] = None,
                 hidden_layers: int = 0, activation_fn=nn.GELU):
        super().__init__()
        from .mlp_layers import Mlp

        hidden_features = 2 * out_features if hidden_features is None else hidden_features
        # ``net.layers`` holds Linear / activation pairs: the key scheme of the reference's checkpoints
        self.net = Mlp(in_features=in_features, hidden_features=[hidden_features] * (hidden_layers + 1),
                       out_features=out_features * 2, act_layer=activation_fn, drop=0.0, final_dropout=False)

    def forward(self, x: Tensor) -> Tuple[Tensor, Tensor]:
        scale, shift = torch.chunk(self.net(x), 2, dim=1)
        return 1 + scale, shift


class ModAFNOMlp(AFNOMlp):
    """``AFNOMlp`` whose hidden activations are scaled / shifted by a modulation embedding."""

    def __init__(self, in_features: int, latent_features: int, out_features: int, mod_features: int,
                 activation_fn: nn.Module = nn.GELU(), drop: float = 0.0, scale_shift_kwargs=None):
        super().__init__(in_features, latent_features, out_features, activation_fn=activation_fn, drop=drop)
        self.scale_shift = ScaleShiftMlp(mod_features, latent_features, **(scale_shift_kwargs or {}))

    def forward(self, x: Tensor, mod_embed: Tensor) -> Tensor:
        scale, shift = self.scale_shift(mod_embed)
        scale, shift = scale.view(-1, 1, 1, scale.shape[1]), shift.view(-1, 1, 1, shift.shape[1])
        x = self.fc1(x)
        x = x * scale + shift
        x = self.drop(self.act(x))
        return self.drop(self.fc2(x))


class ModAFNO2DLayer(AFNO2DLayer):
    """``AFNO2DLayer`` with modulation of the hidden spectral features (``scale_shift_mode`` "complex" or "real")."""

    def __init__(self, hidden_size: int, mod_features: int, num_blocks: int = 8, sparsity_threshold: float = 0.01,
                 hard_thresholding_fraction: float = 1, hidden_size_factor: int = 1, scale_shift_kwargs=None,
                 scale_shift_mode: str = "complex"):
        super().__init__(hidden_size, num_blocks, sparsity_threshold, hard_thresholding_fraction, hidden_size_factor)
        if scale_shift_mode not in ("complex", "real"):
            raise ValueError("scale_shift_mode must be 'real' or 'complex'")
        self.scale_shift_mode = scale_shift_mode
        self.channel_mul = 1 if scale_shift_mode == "real" else 2
        self.scale_shift = ScaleShiftMlp(mod_features, num_blocks * self.block_size * hidden_size_factor * self.channel_mul,
                                         **(scale_shift_kwargs or {}))
        self._mod = None

    def _spectral_mlp(self, xr, xi):
        scale, shift = self._mod
        o1r, o1i = _block_cmul(xr, xi, self.w1, self.b1)
        if self.scale_shift_mode == "real":
            o1r, o1i = o1r * scale + shift, o1i * scale + shift
        else:
            (sr, si), (hr, hi) = scale.chunk(2, dim=-1) if False else (scale[0], scale[1]), (shift[0], shift[1])
            o1r, o1i = o1r * sr - o1i * si + hr, o1i * sr + o1r * si + hi
        o1r, o1i = F.relu(o1r), F.relu(o1i)
        return _block_cmul(o1r, o1i, self.w2, self.b2)

    def forward(self, x: Tensor, mod_embed: Tensor) -> Tensor:
        scale, shift = self.scale_shift(mod_embed)
        B = scale.shape[0]
        shp = (B, 1, 1, self.num_blocks, self.block_size * self.hidden_size_factor)
        if self.scale_shift_mode == "real":
            self._mod = (scale.view(*shp), shift.view(*shp))
        else:
            s = scale.view(B, 1, 1, 2, self.num_blocks, -1)
            h = shift.view(B, 1, 1, 2, self.num_blocks, -1)
            self._mod = ((s[:, :, :, 0], s[:, :, :, 1]), (h[:, :, :, 0], h[:, :, :, 1]))
        try:
            return super().forward(x)
        finally:
            self._mod = None
