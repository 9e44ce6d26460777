"""Space-time diffusion transformer on ``[B, T, X, C]`` tokens with optional temporal and pixel-observation attention.

Counterpart of ``physicsnemo/experimental/models/healda/video_dit.py`` (``VideoDiTBlock`` :59, ``VideoDiT`` :331);
sub-module names are the same.  Every block runs, each behind its own adaptive layer norm and gate: spatial self
attention within a frame, cross attention to packed observation tokens (optional), attention along time per pixel
(optional, space-sharded under context parallelism: the activations are resharded time -> space before and back after),
and the MLP.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from ....core.meta import ModelMetaData
from ....core.module import Module
from ....nn.module.conditioning_embedders import ConditioningEmbedderType, get_conditioning_embedder
from ....nn.module.dit_layers import get_attention, get_layer_norm
from ....nn.module.drop import DropPath
from ....nn.module.mlp_layers import Mlp
from ....nn.module.rope import RotaryEmbedding1DTables
from .adaln import AdaLNModulation, gated_residual, modulate
from .attention_layers import TemporalAttention
from .sharding import shard_t, shard_t_shardtensor, shard_x, shard_x_shardtensor

__all__ = ["VideoDiTBlock", "VideoDiT"]


@dataclass
class MetaData(ModelMetaData):
    amp_gpu: bool = True
    bf16: bool = True


class VideoDiTBlock(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, *, condition_embed_dim: int, attention_backend: Union[str, nn.Module] = "timm",
                 layernorm_backend: str = "torch", mlp_ratio: float = 4.0, norm_eps: float = 1e-6, attn_drop_rate: float = 0.0,
                 proj_drop_rate: float = 0.0, mlp_drop_rate: float = 0.0, final_mlp_dropout: bool = True, drop_path: float = 0.0,
                 temporal_attention: bool = False, use_rope: bool = True, temporal_kwargs: Optional[Dict[str, Any]] = None,
                 cross_attention: Optional[Callable[..., nn.Module]] = None, is_causal: bool = False, adaln_zero_init: bool = True,
                 attn_kwargs: Optional[Dict[str, Any]] = None):
        super().__init__()
        self.hidden_size, self.condition_embed_dim = hidden_size, condition_embed_dim
        norm = lambda: get_layer_norm(hidden_size, layernorm_backend, elementwise_affine=False, eps=norm_eps)  # noqa: E731
        ada = lambda n=1: AdaLNModulation(hidden_size, condition_embed_dim, n_blocks=n, zero_init=adaln_zero_init)  # noqa: E731
        if isinstance(attention_backend, nn.Module):
            self.attention = attention_backend
        else:
            kw = dict(attn_kwargs or {})
            if attention_backend in ("natten2d", "natten2d_rope"):
                kw.setdefault("norm_layer", layernorm_backend)
            self.attention = get_attention(hidden_size=hidden_size, num_heads=num_heads, attention_backend=attention_backend,
                                           attn_drop_rate=attn_drop_rate, proj_drop_rate=proj_drop_rate, **kw)
        self.norm1_modulation = ada(2)                       # spatial attention and MLP share one projection
        self.attn_norm = norm()
        self.linear = Mlp(in_features=hidden_size, hidden_features=int(hidden_size * mlp_ratio), act_layer=lambda: nn.GELU(approximate="tanh"),
                          drop=mlp_drop_rate, final_dropout=final_mlp_dropout)
        self.mlp_norm = norm()
        self.temporal_attention = self.temporal_attn_modulation = self.temporal_attn_norm = None
        if temporal_attention:
            self.temporal_attention = TemporalAttention(hidden_size=hidden_size, num_heads=num_heads, use_rope=use_rope, is_causal=is_causal,
                                                        **(temporal_kwargs or {}))
            self.temporal_attn_modulation, self.temporal_attn_norm = ada(), norm()
        self.cross_attention = cross_attention() if cross_attention is not None else None
        self.cross_attn_modulation = self.cross_attn_norm = None
        if self.cross_attention is not None:
            self.cross_attn_modulation, self.cross_attn_norm = ada(), norm()
        self.drop_path = DropPath(drop_path)
        self._reshard_mode: Optional[str] = None
        self._reshard_target = None

    def initialize_weights(self) -> None:
        for mod in (self.norm1_modulation, self.temporal_attn_modulation, self.cross_attn_modulation):
            if mod is not None:
                mod.initialize_weights()

    def set_context_parallel(self, mode: Optional[str], target=None) -> None:
        """``mode``: ``None`` (no resharding), ``"all_to_all"`` (``target`` = process group) or ``"shardtensor"`` (device mesh)."""
        if mode not in (None, "all_to_all", "shardtensor"):
            raise ValueError(f"unknown reshard mode {mode!r}")
        if mode == "all_to_all" and not isinstance(target, dist.ProcessGroup):
            raise TypeError(f"mode='all_to_all' requires target to be a ProcessGroup, got {type(target).__name__}")
        if mode == "shardtensor":
            from torch.distributed.device_mesh import DeviceMesh

            if not isinstance(target, DeviceMesh):
                raise TypeError(f"mode='shardtensor' requires target to be a DeviceMesh, got {type(target).__name__}")
        self._reshard_mode, self._reshard_target = mode, target

    def _reshard(self, x: torch.Tensor, to_space: bool) -> torch.Tensor:
        if self._reshard_mode == "all_to_all":
            return (shard_x if to_space else shard_t)(x, self._reshard_target)
        if self._reshard_mode == "shardtensor":
            return (shard_x_shardtensor if to_space else shard_t_shardtensor)(x, self._reshard_target)
        return x

    def forward(self, hidden_states: torch.Tensor, c: torch.Tensor, attn_kwargs: Optional[Dict[str, Any]] = None,
                cross_attn_kwargs: Optional[Dict[str, Any]] = None, temporal_attn_kwargs: Optional[Dict[str, Any]] = None) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if hidden_states.ndim != 4:
                raise ValueError(f"Expected hidden_states of shape (B, T, X, C), got {hidden_states.ndim}D tensor with shape "
                                 f"{tuple(hidden_states.shape)}")
            if tuple(c.shape) != (hidden_states.shape[0], self.condition_embed_dim):
                raise ValueError(f"Expected conditioning of shape ({hidden_states.shape[0]}, {self.condition_embed_dim}), got tensor with "
                                 f"shape {tuple(c.shape)}")
            if self.cross_attention is not None and not cross_attn_kwargs:
                raise ValueError("cross_attention was provided at construction but no cross_attn_kwargs was passed to forward")
        b, t, x, ch = hidden_states.shape
        h = hidden_states
        a_shift, a_scale, a_gate, m_shift, m_scale, m_gate = self.norm1_modulation(c)
        spatial = self.attention(modulate(self.attn_norm(h), a_shift, a_scale).reshape(b * t, x, ch), **(attn_kwargs or {}))
        h = gated_residual(h, spatial.reshape(b, t, x, ch), a_gate, self.drop_path)
        if self.cross_attention is not None:
            shift, scale, gate = self.cross_attn_modulation(c)
            h = gated_residual(h, self.cross_attention(modulate(self.cross_attn_norm(h), shift, scale), **cross_attn_kwargs), gate, self.drop_path)
        if self.temporal_attention is not None:
            h = self._reshard(h, to_space=True)
            shift, scale, gate = self.temporal_attn_modulation(c)
            h = gated_residual(h, self.temporal_attention(modulate(self.temporal_attn_norm(h), shift, scale), **(temporal_attn_kwargs or {})),
                               gate, self.drop_path)
            h = self._reshard(h, to_space=False)
        return gated_residual(h, self.linear(modulate(self.mlp_norm(h), m_shift, m_scale)), m_gate, self.drop_path)


class VideoDiT(Module):
    """Tokenizer (must emit ``[B, T, X, hidden]``) -> ``num_layers`` ``VideoDiTBlock`` -> detokenizer, conditioned on the
    noise level (and an optional vector) through a conditioning embedder."""

    def __init__(self, tokenizer: nn.Module, detokenizer: nn.Module, hidden_size: int, num_heads: int, num_layers: int, *,
                 emb_channels: Optional[int] = None, noise_channels: Optional[int] = None, condition_dim: int = 0,
                 temporal_attention: bool = False, use_rope: bool = True, rope_base: int = 100, max_seq_len: int = 100,
                 temporal_kwargs: Optional[Dict[str, Any]] = None, cross_attention: Optional[Callable[..., nn.Module]] = None,
                 is_causal: bool = False, attention_backend: Union[str, nn.Module] = "timm", layernorm_backend: str = "torch",
                 mlp_ratio: float = 4.0, drop_path: float = 0.0, drop_path_rates: Optional[List[float]] = None,
                 conditioning_embedder: Any = "edm", conditioning_embedder_kwargs: Optional[Dict[str, Any]] = None,
                 dit_initialization: bool = True, adaln_zero_init: bool = True, attn_kwargs: Optional[Dict[str, Any]] = None,
                 block_kwargs: Optional[Dict[str, Any]] = None):
        super().__init__(meta=MetaData())
        self.tokenizer, self.detokenizer, self.hidden_size, self.condition_dim = tokenizer, detokenizer, hidden_size, condition_dim
        if isinstance(conditioning_embedder, str):
            kind = ConditioningEmbedderType[conditioning_embedder.upper()]
            kw = dict(conditioning_embedder_kwargs or {})
            if kind is ConditioningEmbedderType.EDM:
                kw.setdefault("emb_channels", emb_channels or 4 * hidden_size)
                kw.setdefault("noise_channels", noise_channels or hidden_size)
            self.conditioning_embedder = get_conditioning_embedder(kind, hidden_size=hidden_size, condition_dim=condition_dim,
                                                                   amp_mode=self.meta.amp_gpu, **kw)
        elif hasattr(conditioning_embedder, "output_dim") and callable(conditioning_embedder):
            self.conditioning_embedder = conditioning_embedder
        else:
            raise TypeError("conditioning_embedder must be a name in {'dit', 'edm', 'zero'} or a ConditioningEmbedder instance")
        cond_dim = self.conditioning_embedder.output_dim
        self.temporal_rope = (RotaryEmbedding1DTables(head_dim=hidden_size // num_heads, max_seq_len=max_seq_len, theta=rope_base)
                              if temporal_attention and use_rope else None)
        if drop_path_rates is None:
            drop_path_rates = [drop_path * i / max(1, num_layers - 1) for i in range(num_layers)]
        elif len(drop_path_rates) != num_layers:
            raise ValueError(f"drop_path_rates length ({len(drop_path_rates)}) must match num_layers ({num_layers})")
        self.blocks = nn.ModuleList(
            VideoDiTBlock(hidden_size, num_heads, condition_embed_dim=cond_dim, attention_backend=attention_backend,
                          layernorm_backend=layernorm_backend, mlp_ratio=mlp_ratio, drop_path=drop_path_rates[i],
                          temporal_attention=temporal_attention, use_rope=use_rope, temporal_kwargs=temporal_kwargs,
                          cross_attention=cross_attention, is_causal=is_causal, adaln_zero_init=adaln_zero_init, attn_kwargs=attn_kwargs,
                          **(block_kwargs or {})) for i in range(num_layers))
        if dit_initialization:
            self.initialize_weights()

    def initialize_weights(self) -> None:
        def basic(m):
            if isinstance(m, nn.Linear):
                nn.init.xavier_uniform_(m.weight)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

        self.apply(basic)
        for m in (self.tokenizer, self.detokenizer, *self.blocks):
            if hasattr(m, "initialize_weights"):
                m.initialize_weights()

    def set_context_parallel(self, mode: Optional[str], target=None) -> None:
        for blk in self.blocks:
            blk.set_context_parallel(mode, target)

    def forward(self, x: torch.Tensor, t: torch.Tensor, condition: Optional[torch.Tensor] = None, attn_kwargs: Optional[Dict[str, Any]] = None,
                cross_attn_kwargs: Optional[Dict[str, Any]] = None, temporal_attn_kwargs: Optional[Dict[str, Any]] = None,
                tokenizer_kwargs: Optional[Dict[str, Any]] = None) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if x.ndim != 4:
                raise ValueError(f"Expected 4D input (B, C, T, X), got {x.ndim}D tensor with shape {tuple(x.shape)}")
            if t.ndim != 1 or t.shape[0] != x.shape[0]:
                raise ValueError(f"Expected t of shape ({x.shape[0]},), got tensor with shape {tuple(t.shape)}")
            if condition is not None and tuple(condition.shape) != (x.shape[0], self.condition_dim):
                raise ValueError(f"Expected condition of shape ({x.shape[0]}, {self.condition_dim}), got tensor with shape "
                                 f"{tuple(condition.shape)}")
        h = self.tokenizer(x, **(tokenizer_kwargs or {}))
        if not torch.compiler.is_compiling() and h.ndim != 4:
            raise ValueError(f"tokenizer must emit (B, T, X, hidden) for VideoDiT; got {h.ndim}D (use a tokenizer with "
                             "separate_time_axis=True).")
        emb = self.conditioning_embedder(t, condition=condition)
        tkw = dict(temporal_attn_kwargs or {})
        if self.temporal_rope is not None:
            tkw["rope_cos"], tkw["rope_sin"] = self.temporal_rope(seq_len=h.shape[1])
        for blk in self.blocks:
            h = blk(h, emb, attn_kwargs=attn_kwargs, cross_attn_kwargs=cross_attn_kwargs, temporal_attn_kwargs=tkw)
        return self.detokenizer(h, emb)
