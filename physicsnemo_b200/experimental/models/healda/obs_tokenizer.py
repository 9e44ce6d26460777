"""FiLM tokenizer of scalar observations: ``token = alpha(meta) * obs + beta(meta)``.

Counterpart of ``physicsnemo/experimental/models/healda/obs_tokenizer.py`` (``ObsTokenizerFiLM`` :111) and of its fused
Triton forward / backward (``kernels/obs_tokenizer_film.py``).  The conditioning MLP is
``Linear(cat[meta, E_type[id], E_chan[ch], E_plat[pl]]) -> LayerNorm -> SiLU -> Linear -> (alpha, beta)``.

The first linear layer is re-associated per step: the embedding tables are multiplied by their slice of the weight once
(``[n_embed, hidden]``, a tiny GEMM), so that per observation the layer is three table-row gathers plus a
``meta_dim x hidden`` product; the concatenated conditioning matrix ``[nobs, cond_dim]`` and its skinny-K GEMM are never
formed.  Only rows that occur are touched in the backward (``index_add`` into the projected tables).  The second linear
layer is a regular GEMM (``K = hidden``) and goes through ``nn.Linear``.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

__all__ = ["ObsTokenizerFiLM", "GLOBAL_MAX_CHANNELS", "GLOBAL_MAX_PLATFORM"]

GLOBAL_MAX_CHANNELS = 1024
GLOBAL_MAX_PLATFORM = 1024


def _default_film_hidden_dim(out_dim: int) -> int:
    return out_dim * 2 if out_dim <= 64 else out_dim


class ObsTokenizerFiLM(torch.nn.Module):
    def __init__(self, meta_dim: int, out_dim: int, n_embed: int = 1024, obs_type_embed_dim: int = 4,
                 channel_embed_dim: Optional[int] = None, platform_embed_dim: Optional[int] = None, use_fused_mlp: bool = True,
                 hidden_dim: Optional[int] = None):
        super().__init__()
        channel_embed_dim = obs_type_embed_dim if channel_embed_dim is None else channel_embed_dim
        platform_embed_dim = 0 if platform_embed_dim is None else platform_embed_dim
        hidden_dim = _default_film_hidden_dim(out_dim) if hidden_dim is None else hidden_dim
        if hidden_dim <= 0:
            raise ValueError(f"hidden_dim must be positive, got {hidden_dim}")
        self.meta_dim, self.out_dim, self.hidden_dim = meta_dim, out_dim, hidden_dim
        self.obs_type_embed_dim, self.channel_embed_dim, self.platform_embed_dim = obs_type_embed_dim, channel_embed_dim, platform_embed_dim
        self.use_platform_embedding = platform_embed_dim > 0
        self.use_fused_mlp = use_fused_mlp            # True: re-associated first layer; False: concatenate and multiply
        self.embed_table = torch.nn.Embedding(n_embed, obs_type_embed_dim)
        self.channel_embedding = torch.nn.Embedding(GLOBAL_MAX_CHANNELS, channel_embed_dim)
        self.platform_embedding = torch.nn.Embedding(GLOBAL_MAX_PLATFORM, platform_embed_dim) if self.use_platform_embedding else None
        cond_dim = meta_dim + obs_type_embed_dim + channel_embed_dim + platform_embed_dim
        self.cond_mlp = torch.nn.Sequential(torch.nn.Linear(cond_dim, hidden_dim), torch.nn.LayerNorm(hidden_dim), torch.nn.SiLU(),
                                            torch.nn.Linear(hidden_dim, 2 * out_dim))

    def _build_conditioning(self, float_metadata, obs_type, channel_ids, platform_ids) -> torch.Tensor:
        parts = [float_metadata, self.embed_table(obs_type), self.channel_embedding(channel_ids)]
        if self.use_platform_embedding:
            if platform_ids is None:
                raise ValueError("platform embedding requires platform ids")
            parts.append(self.platform_embedding(platform_ids))
        return torch.cat(parts, dim=-1)

    def _first_layer(self, float_metadata, obs_type, channel_ids, platform_ids) -> torch.Tensor:
        lin = self.cond_mlp[0]
        w_meta, w_type, w_chan, w_plat = lin.weight.split([self.meta_dim, self.obs_type_embed_dim, self.channel_embed_dim,
                                                           self.platform_embed_dim], dim=1)
        dt = float_metadata.dtype
        pre = F.linear(float_metadata, w_meta.to(dt), lin.bias.to(dt))
        pre = pre + (self.embed_table.weight @ w_type.t()).to(dt)[obs_type] + (self.channel_embedding.weight @ w_chan.t()).to(dt)[channel_ids]
        if self.use_platform_embedding:
            pre = pre + (self.platform_embedding.weight @ w_plat.t()).to(dt)[platform_ids]
        return pre

    def forward(self, obs: torch.Tensor, float_metadata: torch.Tensor, obs_type: torch.Tensor, channel_ids: torch.Tensor,
                platform_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if obs.ndim != 1:
                raise ValueError(f"Expected obs of shape (nobs,), got {obs.ndim}D tensor with shape {tuple(obs.shape)}")
            nobs = obs.shape[0]
            if float_metadata.ndim != 2 or float_metadata.shape[0] != nobs:
                raise ValueError(f"Expected float_metadata of shape ({nobs}, meta_dim), got tensor with shape {tuple(float_metadata.shape)}")
            if float_metadata.shape[1] != self.meta_dim:
                raise ValueError(f"Expected float_metadata with meta_dim {self.meta_dim}, got {float_metadata.shape[1]}")
            for name, t in (("obs_type", obs_type), ("channel_ids", channel_ids)):
                if t.ndim != 1 or t.shape[0] != nobs:
                    raise ValueError(f"Expected {name} of shape ({nobs},) matching obs, got tensor with shape {tuple(t.shape)}")
            if self.use_platform_embedding:
                if platform_ids is None:
                    raise ValueError("platform_ids required when platform embedding is enabled")
                if platform_ids.ndim != 1 or platform_ids.shape[0] != nobs:
                    raise ValueError(f"Expected platform_ids of shape ({nobs},) matching obs, got tensor with shape "
                                     f"{tuple(platform_ids.shape)}")
        if self.use_fused_mlp:
            pre = self._first_layer(float_metadata, obs_type, channel_ids, platform_ids)
        else:
            pre = self.cond_mlp[0](self._build_conditioning(float_metadata, obs_type, channel_ids, platform_ids))
        alpha, beta = self.cond_mlp[3](self.cond_mlp[2](self.cond_mlp[1](pre))).chunk(2, dim=-1)
        return torch.addcmul(beta, alpha, obs.unsqueeze(-1))
