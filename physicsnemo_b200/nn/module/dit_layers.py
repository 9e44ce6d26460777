"""Diffusion-transformer building blocks.

Parity: ``physicsnemo/nn/module/dit_layers.py`` — attention back-ends (``"timm"``: plain multi-head
self-attention with timm's parameter names ``qkv / q_norm / k_norm / proj``; ``"natten2d"`` /
``"natten2d_rope"``: 2-D neighbourhood attention, optionally with axial RoPE and a learned mask token;
``"transformer_engine"`` is not available in this build and raises), ``PerSampleDropout``, the adaLN-Zero
``DiTBlock``, ``ProjLayer``, and the tokenizer / detokenizer families with their factories.
"""
from abc import ABC, abstractmethod
from typing import Any, Dict, Literal, Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...core import Module
from ..functional.natten import na2d as _na2d_func
from .drop import DropPath
from .mlp_layers import Mlp
from .rope import apply_rotary_pos_emb
from .utils import PatchEmbed2D


class RmsNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, affine: bool = True):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim)) if affine else None

    def forward(self, x):
        y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)
        y = y.to(x.dtype)
        return y * self.weight if self.weight is not None else y


def get_layer_norm(hidden_size: int, layernorm_backend: Literal["apex", "torch"], elementwise_affine: bool = False,
                   eps: float = 1e-6) -> nn.Module:
    if layernorm_backend == "apex":
        raise ImportError("Apex is not available. Please install Apex to use FusedLayerNorm or choose 'torch'.")
    if layernorm_backend == "torch":
        return nn.LayerNorm(hidden_size, elementwise_affine=elementwise_affine, eps=eps)
    raise ValueError("layernorm_backend must be one of 'apex' or 'torch'.")


class AttentionModuleBase(Module, ABC):
    @abstractmethod
    def forward(self, x):
        ...


class _Attention(nn.Module):
    """Multi-head self-attention with the parameter layout of ``timm.layers.attention.Attention``."""

    def __init__(self, dim, num_heads, qkv_bias=True, qk_norm=False, attn_drop=0.0, proj_drop=0.0, norm_layer=None, **_):
        super().__init__()
        if dim % num_heads:
            raise ValueError("dim should be divisible by num_heads")
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.q_norm = norm_layer(self.head_dim) if qk_norm else nn.Identity()
        self.k_norm = norm_layer(self.head_dim) if qk_norm else nn.Identity()
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj = nn.Linear(dim, dim)
        self.proj_drop = nn.Dropout(proj_drop)

    def forward(self, x, attn_mask=None, is_causal=False):
        B, N, C = x.shape
        q, k, v = self.qkv(x).reshape(B, N, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        q, k = self.q_norm(q), self.k_norm(k)
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, is_causal=is_causal,
                                             dropout_p=self.attn_drop.p if self.training else 0.0)
        return self.proj_drop(self.proj(out.transpose(1, 2).reshape(B, N, C)))


class TimmSelfAttention(AttentionModuleBase):
    def __init__(self, hidden_size: int, num_heads: int, attn_drop_rate: float = 0.0, proj_drop_rate: float = 0.0,
                 qk_norm_type: Literal["RMSNorm", "LayerNorm"] | None = None, qk_norm_affine: bool = True,
                 is_causal: bool = False, **kwargs: Any):
        super().__init__()
        self.is_causal = is_causal
        if qk_norm_type == "RMSNorm":
            kwargs.update(qk_norm=True, norm_layer=lambda d: RmsNorm(d, affine=qk_norm_affine))
        elif qk_norm_type == "LayerNorm":
            kwargs.update(qk_norm=True, norm_layer=lambda d: nn.LayerNorm(d, elementwise_affine=qk_norm_affine))
        self.attn_op = _Attention(dim=hidden_size, num_heads=num_heads, attn_drop=attn_drop_rate,
                                  proj_drop=proj_drop_rate, qkv_bias=True, **kwargs)

    def forward(self, x, attn_mask=None):
        if attn_mask is not None and self.is_causal:
            raise ValueError("attn_mask cannot be combined with is_causal=True in TimmSelfAttention; "
                             "they are mutually exclusive.")
        return self.attn_op(x, attn_mask=attn_mask, is_causal=self.is_causal)


class TESelfAttention(AttentionModuleBase):
    def __init__(self, *args, **kwargs):
        raise ImportError("Transformer Engine is not installed. Please install it with `pip install transformer-engine`.")

    def forward(self, x):  # pragma: no cover
        raise NotImplementedError


class Natten2DSelfAttention(AttentionModuleBase):
    """2-D neighbourhood self-attention on a ``latent_hw`` token lattice given as a flat sequence."""

    def __init__(self, hidden_size: int, num_heads: int, attn_kernel: int = 3, qkv_bias: bool = True, qk_norm: bool = False,
                 attn_drop_rate: float = 0.0, proj_drop_rate: float = 0.0, norm_layer: Literal["apex", "torch"] = "torch",
                 na2d_kwargs: Optional[Dict[str, Any]] = None, use_mask_token: bool = False):
        super().__init__()
        if hidden_size % num_heads != 0:
            raise ValueError("hidden_size should be divisible by num_heads")
        self.num_heads, self.head_dim = num_heads, hidden_size // num_heads
        self.scale = self.head_dim ** -0.5
        self.attn_drop_rate, self.proj_drop_rate, self.norm_layer = attn_drop_rate, proj_drop_rate, norm_layer
        self.attn_kernel = attn_kernel
        self.na2d_kwargs = na2d_kwargs if na2d_kwargs is not None else {}
        self.mask_token = nn.Parameter(torch.zeros(1, 1, hidden_size)) if use_mask_token else None
        self.qkv = nn.Linear(hidden_size, hidden_size * 3, bias=qkv_bias)
        self.q_norm = get_layer_norm(self.head_dim, norm_layer) if qk_norm else nn.Identity()
        self.k_norm = get_layer_norm(self.head_dim, norm_layer) if qk_norm else nn.Identity()
        self.proj = nn.Linear(hidden_size, hidden_size)
        self.attn_drop = nn.Dropout(attn_drop_rate)
        self.proj_drop = nn.Dropout(proj_drop_rate)

    def _apply_mask_token(self, x, invalid_token_mask):
        if self.mask_token is None or invalid_token_mask is None:
            return x
        a = invalid_token_mask.to(dtype=x.dtype)
        a = a.view(1, -1, 1) if a.ndim == 1 else a.unsqueeze(-1)
        return x * (1.0 - a) + self.mask_token.to(x.dtype) * a

    def _qkv(self, x, latent_hw, invalid_token_mask):
        B, N, _ = x.shape
        h, w = int(latent_hw[0]), int(latent_hw[1])
        if not torch.compiler.is_compiling() and N != h * w:
            raise ValueError(f"Sequence length must be {h * w} based on latent_hw={latent_hw}, but got {N}")
        x = self._apply_mask_token(x, invalid_token_mask)
        q, k, v = self.qkv(x).reshape(B, N, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        return self.q_norm(q), self.k_norm(k), v, h, w

    def _finish(self, q, k, v, B, N):
        out = self.attn_drop(_na2d_func(q, k, v, kernel_size=self.attn_kernel, **self.na2d_kwargs))
        return self.proj_drop(self.proj(out.reshape(B, N, -1)))

    def forward(self, x, latent_hw: Tuple[int, int], invalid_token_mask=None):
        B, N, _ = x.shape
        q, k, v, h, w = self._qkv(x, latent_hw, invalid_token_mask)
        to_grid = lambda t: t.permute(0, 2, 1, 3).reshape(B, h, w, self.num_heads, self.head_dim)  # noqa: E731
        return self._finish(to_grid(q), to_grid(k), to_grid(v), B, N)


class RopeNatten2DSelfAttention(Natten2DSelfAttention):
    def __init__(self, *args: Any, **kwargs: Any):
        super().__init__(*args, **kwargs)
        if self.head_dim % 4 != 0:
            raise ValueError(f"head_dim={self.head_dim} must be divisible by 4 for axial 2D RoPE.")

    def forward(self, x, latent_hw: Tuple[int, int], rope_cos, rope_sin, invalid_token_mask=None):
        B, N, _ = x.shape
        q, k, v, h, w = self._qkv(x, latent_hw, invalid_token_mask)
        if not torch.compiler.is_compiling():
            want = (h, w, self.head_dim)
            if tuple(rope_cos.shape) != want or tuple(rope_sin.shape) != want:
                raise ValueError(f"Expected rope_cos/rope_sin of shape {want}, but got "
                                 f"rope_cos={tuple(rope_cos.shape)}, rope_sin={tuple(rope_sin.shape)}")
        shape5 = (B, self.num_heads, h, w, self.head_dim)
        q = apply_rotary_pos_emb(q.reshape(shape5), rope_cos[None, None], rope_sin[None, None]).permute(0, 2, 3, 1, 4)
        k = apply_rotary_pos_emb(k.reshape(shape5), rope_cos[None, None], rope_sin[None, None]).permute(0, 2, 3, 1, 4)
        v = v.reshape(shape5).permute(0, 2, 3, 1, 4)
        return self._finish(q.contiguous(), k.contiguous(), v, B, N)


def get_attention(hidden_size: int, num_heads: int,
                  attention_backend: Literal["transformer_engine", "timm", "natten2d", "natten2d_rope"],
                  attn_drop_rate: float = 0.0, proj_drop_rate: float = 0.0, **attn_kwargs: Any) -> Module:
    table = {"timm": TimmSelfAttention, "transformer_engine": TESelfAttention, "natten2d": Natten2DSelfAttention,
             "natten2d_rope": RopeNatten2DSelfAttention}
    if attention_backend not in table:
        raise ValueError("attention_backend must be one of 'timm', 'transformer_engine', 'natten2d', 'natten2d_rope' "
                         "if using pre-defined attention modules.")
    return table[attention_backend](hidden_size, num_heads, attn_drop_rate=attn_drop_rate, proj_drop_rate=proj_drop_rate,
                                    **attn_kwargs)


class PerSampleDropout(nn.Module):
    """Dropout whose probability may differ per sample of the batch (``p``: float or ``[batch]`` tensor)."""

    def __init__(self, inplace: bool = False):
        super().__init__()
        self.inplace = inplace

    def forward(self, x, p=None):
        if not self.training or p is None:
            return x
        if torch.is_tensor(p) and p.ndim == 0:
            p = float(p.item())
        if isinstance(p, (float, int)):
            return x if p <= 0.0 else F.dropout(x, p=float(p), training=True, inplace=self.inplace)
        if not torch.is_tensor(p):
            raise TypeError("p must be a float, int, or torch.Tensor")
        if p.numel() != x.size(0):
            raise ValueError(f"Per-sample dropout expects p with numel == batch size ({x.size(0)}), got shape {tuple(p.shape)}")
        keep = (1.0 - p.view([-1] + [1] * (x.ndim - 1)).to(device=x.device, dtype=x.dtype)).clamp(min=1e-6)
        mask = (torch.rand_like(x) < keep).to(x.dtype) / keep
        return x.mul_(mask) if self.inplace else x * mask


def _modulate(x, scale, shift):
    return x * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


class DiTBlock(nn.Module):
    """adaLN-Zero transformer block: the condition produces (shift, scale, gate) for the attention and MLP branches."""

    def __init__(self, hidden_size: int, num_heads: int,
                 attention_backend: Union[Literal["transformer_engine", "timm", "natten2d", "natten2d_rope"], Module] = "timm",
                 layernorm_backend: Literal["apex", "torch"] = "torch", norm_eps: float = 1e-6, mlp_ratio: float = 4.0,
                 intermediate_dropout: bool = False, attn_drop_rate: float = 0.0, proj_drop_rate: float = 0.0,
                 mlp_drop_rate: float = 0.0, final_mlp_dropout: bool = True, drop_path: float = 0.0,
                 condition_embed_dim: Optional[int] = None, **attn_kwargs: Any):
        super().__init__()
        if isinstance(attention_backend, nn.Module):
            self.attention = attention_backend
        else:
            kw = dict(attn_kwargs)
            if attention_backend in ("natten2d", "natten2d_rope"):
                kw.setdefault("norm_layer", layernorm_backend)
            self.attention = get_attention(hidden_size=hidden_size, num_heads=num_heads, attention_backend=attention_backend,
                                           attn_drop_rate=attn_drop_rate, proj_drop_rate=proj_drop_rate, **kw)
        self.pre_attention_norm = get_layer_norm(hidden_size, layernorm_backend, elementwise_affine=False, eps=norm_eps)
        self.pre_mlp_norm = get_layer_norm(hidden_size, layernorm_backend, elementwise_affine=False, eps=norm_eps)
        self.interdrop = PerSampleDropout() if intermediate_dropout else None
        self.linear = Mlp(in_features=hidden_size, hidden_features=int(hidden_size * mlp_ratio),
                          act_layer=lambda: nn.GELU(approximate="tanh"), drop=mlp_drop_rate, final_dropout=final_mlp_dropout)
        cond = hidden_size if condition_embed_dim is None else condition_embed_dim
        self.adaptive_modulation = nn.Sequential(nn.SiLU(), nn.Linear(cond, 6 * hidden_size, bias=True))
        self.modulation = _modulate
        self.drop_path = DropPath(drop_path)

    def initialize_weights(self):
        nn.init.constant_(self.adaptive_modulation[-1].weight, 0)
        nn.init.constant_(self.adaptive_modulation[-1].bias, 0)

    def forward(self, x, c, attn_kwargs: Optional[Dict[str, Any]] = None, p_dropout=None):
        a_shift, a_scale, a_gate, m_shift, m_scale, m_gate = self.adaptive_modulation(c).chunk(6, dim=1)
        h = _modulate(self.pre_attention_norm(x), a_scale, a_shift)
        if self.interdrop is not None:
            h = self.interdrop(h, p_dropout)
        elif p_dropout is not None:
            raise ValueError("p_dropout passed to DiTBlock but intermediate_dropout is disabled")
        x = torch.addcmul(x, self.drop_path(a_gate.unsqueeze(1)), self.attention(h, **(attn_kwargs or {})))
        h = self.linear(_modulate(self.pre_mlp_norm(x), m_scale, m_shift))
        return torch.addcmul(x, self.drop_path(m_gate.unsqueeze(1)), h)


class ProjLayer(nn.Module):
    """Final adaLN modulation and linear projection of the tokens."""

    def __init__(self, hidden_size: int, emb_channels: int, layernorm_backend: Literal["apex", "torch"] = "torch"):
        super().__init__()
        self.proj_layer_norm = get_layer_norm(hidden_size, layernorm_backend, elementwise_affine=False, eps=1e-6)
        self.output_projection = nn.Linear(hidden_size, emb_channels, bias=True)
        self.adaptive_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size, 2 * hidden_size, bias=True))
        self.modulation = _modulate

    def forward(self, x, c):
        shift, scale = self.adaptive_modulation(c).chunk(2, dim=1)
        return self.output_projection(_modulate(self.proj_layer_norm(x), scale, shift))


class TokenizerModuleBase(Module, ABC):
    @abstractmethod
    def forward(self, x):
        ...

    @abstractmethod
    def initialize_weights(self):
        ...


class PatchEmbed2DTokenizer(TokenizerModuleBase):
    def __init__(self, input_size: Tuple[int, int], patch_size: Tuple[int, int], in_channels: int, hidden_size: int,
                 pos_embed: str = "learnable", **tokenizer_kwargs: Any):
        super().__init__()
        self.input_size, self.patch_size = input_size, patch_size
        self.in_channels, self.hidden_size = in_channels, hidden_size
        self.h_patches, self.w_patches = input_size[0] // patch_size[0], input_size[1] // patch_size[1]
        self.num_patches = self.h_patches * self.w_patches
        self.x_embedder = PatchEmbed2D(input_size, patch_size, in_channels, hidden_size, **tokenizer_kwargs)
        self.pos_embed = nn.Parameter(torch.zeros(1, self.num_patches, hidden_size)) if pos_embed == "learnable" else 0.0

    def initialize_weights(self):
        w = self.x_embedder.proj.weight.data
        nn.init.xavier_uniform_(w.view([w.shape[0], -1]))
        if self.x_embedder.proj.bias is not None:
            nn.init.constant_(self.x_embedder.proj.bias, 0)
        if isinstance(self.pos_embed, nn.Parameter):
            nn.init.normal_(self.pos_embed, std=0.02)

    def forward(self, x):
        return self.x_embedder(x).flatten(2).transpose(1, 2) + self.pos_embed


def get_tokenizer(input_size, patch_size, in_channels: int, hidden_size: int,
                  tokenizer: Literal["patch_embed_2d", "hpx_patch_embed"] = "patch_embed_2d", **tokenizer_kwargs: Any):
    if tokenizer == "patch_embed_2d":
        return PatchEmbed2DTokenizer(input_size=input_size, patch_size=patch_size, in_channels=in_channels,
                                     hidden_size=hidden_size, **tokenizer_kwargs)
    if tokenizer == "hpx_patch_embed":
        from .hpx.tokenizer import HEALPixPatchTokenizer

        return HEALPixPatchTokenizer(in_channels=in_channels, hidden_size=hidden_size, **tokenizer_kwargs)
    raise ValueError("tokenizer must be 'patch_embed_2d' or 'hpx_patch_embed'.")


class DetokenizerModuleBase(Module, ABC):
    @abstractmethod
    def forward(self, x_tokens, c):
        ...

    @abstractmethod
    def initialize_weights(self):
        ...


class ProjReshape2DDetokenizer(DetokenizerModuleBase):
    def __init__(self, input_size: Tuple[int, int], patch_size: Tuple[int, int], out_channels: int, hidden_size: int,
                 layernorm_backend: Literal["apex", "torch"] = "torch"):
        super().__init__()
        self.input_size, self.patch_size = input_size, patch_size
        self.out_channels, self.hidden_size = out_channels, hidden_size
        self.h_patches, self.w_patches = input_size[0] // patch_size[0], input_size[1] // patch_size[1]
        self.proj_layer = ProjLayer(hidden_size=hidden_size, emb_channels=patch_size[0] * patch_size[1] * out_channels,
                                    layernorm_backend=layernorm_backend)

    def initialize_weights(self):
        for t in (self.proj_layer.adaptive_modulation[-1].weight, self.proj_layer.adaptive_modulation[-1].bias,
                  self.proj_layer.output_projection.weight, self.proj_layer.output_projection.bias):
            nn.init.constant_(t, 0)

    def forward(self, x_tokens, c):
        p0, p1 = self.patch_size
        x = self.proj_layer(x_tokens, c).reshape(-1, self.h_patches, self.w_patches, p0, p1, self.out_channels)
        return x.permute(0, 5, 1, 3, 2, 4).reshape(-1, self.out_channels, self.h_patches * p0, self.w_patches * p1)


class ConvDetokenizer(DetokenizerModuleBase):
    """``ProjReshape2DDetokenizer`` followed by a residual convolutional smoothing head (zero-initialised)."""

    def __init__(self, input_size: Tuple[int, int], patch_size: Tuple[int, int], out_channels: int, hidden_size: int,
                 layernorm_backend: Literal["apex", "torch"] = "torch", conv_layers: int = 2, conv_hidden: int = 64,
                 conv_kernel: int = 3):
        super().__init__()
        self.proj = ProjReshape2DDetokenizer(input_size=input_size, patch_size=patch_size, out_channels=out_channels,
                                             hidden_size=hidden_size, layernorm_backend=layernorm_backend)
        if conv_layers < 1:
            raise ValueError(f"conv_layers must be >= 1; got {conv_layers}")
        layers, c_in = [], out_channels
        for i in range(int(conv_layers)):
            last = i == conv_layers - 1
            c_out = out_channels if last else conv_hidden
            layers.append(nn.Conv2d(c_in, c_out, conv_kernel, padding=conv_kernel // 2))
            if not last:
                layers.append(nn.GELU())
            c_in = c_out
        self.conv_head = nn.Sequential(*layers)

    def initialize_weights(self) -> None:
        self.proj.initialize_weights()
        last = [m for m in self.conv_head if isinstance(m, nn.Conv2d)][-1]
        nn.init.zeros_(last.weight)
        if last.bias is not None:
            nn.init.zeros_(last.bias)

    def forward(self, x_tokens, c):
        img = self.proj(x_tokens, c)
        return img + self.conv_head(img)


def get_detokenizer(input_size, patch_size, out_channels: int, hidden_size: int,
                    detokenizer: Literal["proj_reshape_2d", "proj_reshape_2d_conv", "hpx_patch_detokenizer"] = "proj_reshape_2d",
                    **detokenizer_kwargs: Any):
    if detokenizer == "proj_reshape_2d":
        return ProjReshape2DDetokenizer(input_size=input_size, patch_size=patch_size, out_channels=out_channels,
                                        hidden_size=hidden_size, **detokenizer_kwargs)
    if detokenizer == "proj_reshape_2d_conv":
        return ConvDetokenizer(input_size=input_size, patch_size=patch_size, out_channels=out_channels,
                               hidden_size=hidden_size, **detokenizer_kwargs)
    if detokenizer == "hpx_patch_detokenizer":
        from .hpx.tokenizer import HEALPixPatchDetokenizer

        return HEALPixPatchDetokenizer(hidden_size=hidden_size, out_channels=out_channels, **detokenizer_kwargs)
    raise ValueError("detokenizer must be 'proj_reshape_2d', 'proj_reshape_2d_conv', or 'hpx_patch_detokenizer'.")
