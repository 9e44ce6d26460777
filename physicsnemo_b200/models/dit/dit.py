"""Diffusion transformer (DiT).

Parity: ``physicsnemo/models/dit/dit.py`` — tokenizer → conditioning embedder (timestep [+ condition]) → ``depth``
adaLN-Zero ``DiTBlock``s → detokenizer; attention back-ends ``timm`` (dense) and ``natten2d`` / ``natten2d_rope``
(neighbourhood attention on the latent lattice, optional rotary embeddings and learned tokens for invalid
pixels); legacy checkpoints (``t_embedder.*``) are migrated on load.
"""
import warnings
from dataclasses import dataclass
from typing import Any, Dict, Literal, Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.conditioning_embedders import ConditioningEmbedder, ConditioningEmbedderType, get_conditioning_embedder
from ...nn.module.dit_layers import (DetokenizerModuleBase, DiTBlock, TokenizerModuleBase, get_detokenizer,
                                     get_tokenizer)
from ...nn.module.rope import RotaryEmbedding2DTables

_ATTN = ("timm", "transformer_engine", "natten2d", "natten2d_rope")


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp_cpu: bool = False
    amp_gpu: bool = True
    torch_fx: bool = False
    bf16: bool = True
    onnx: bool = False
    func_torch: bool = False
    auto_grad: bool = False


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


class DiT(Module):
    __model_checkpoint_version__ = "0.2.0"
    __supported_model_checkpoint_version__ = {
        "0.1.0": "Automatically converting legacy DiT checkpoint timestep / conditioning embedder arguments.",
    }

    @classmethod
    def _backward_compat_arg_mapper(cls, version: str, args: Dict[str, Any]) -> Dict[str, Any]:
        args = super()._backward_compat_arg_mapper(version, args)
        if version == "0.1.0" and "timestep_embed_kwargs" in args:
            args["conditioning_embedder_kwargs"] = args.pop("timestep_embed_kwargs")
        return args

    def __init__(self, input_size, in_channels: int, patch_size=(8, 8),
                 tokenizer: Union[Literal["patch_embed_2d", "hpx_patch_embed"], Module] = "patch_embed_2d",
                 detokenizer: Union[Literal["proj_reshape_2d", "proj_reshape_2d_conv", "hpx_patch_detokenizer"], Module] = "proj_reshape_2d",
                 out_channels: Optional[int] = None, hidden_size: int = 384, depth: int = 12, num_heads: int = 8,
                 mlp_ratio: float = 4.0, attention_backend: str = "timm", layernorm_backend: str = "torch",
                 condition_dim: Optional[int] = None, conditioning_embedder="dit", dit_initialization: Optional[int] = True,
                 conditioning_embedder_kwargs: Dict[str, Any] = {}, tokenizer_kwargs: Dict[str, Any] = {},
                 detokenizer_kwargs: Dict[str, Any] = {}, block_kwargs: Dict[str, Any] = {}, attn_kwargs: Dict[str, Any] = {},
                 drop_path_rates: list[float] | None = None, force_tokenization_fp32: bool = False,
                 use_nan_mask_tokens: bool = False):
        super().__init__(meta=MetaData())
        self.input_size, self.patch_size = _pair(input_size), _pair(patch_size)
        self.in_channels, self.out_channels = in_channels, out_channels or in_channels
        self.num_heads, self.condition_dim = num_heads, condition_dim
        if attention_backend not in _ATTN:
            raise ValueError("attention_backend must be one of 'timm', 'transformer_engine', 'natten2d', 'natten2d_rope'")
        if layernorm_backend not in ("apex", "torch"):
            raise ValueError("layernorm_backend must be one of 'apex', 'torch'")
        natten = attention_backend in ("natten2d", "natten2d_rope")
        latent_hw = (self.input_size[0] // self.patch_size[0], self.input_size[1] // self.patch_size[1]) if natten else None
        self._latent_h, self._latent_w = latent_hw if natten else (None, None)
        self.attn_kwargs_forward = {"latent_hw": latent_hw} if natten else {}
        self._use_nan_mask_tokens = use_nan_mask_tokens
        if use_nan_mask_tokens and not natten:
            raise ValueError("use_nan_mask_tokens=True requires a NATTEN attention backend ('natten2d' or 'natten2d_rope')")
        attn_kwargs = dict(attn_kwargs)
        self._is_rope = attention_backend == "natten2d_rope"
        self.rope = None
        if self._is_rope:
            self.rope = RotaryEmbedding2DTables(head_dim=hidden_size // num_heads, latent_hw=latent_hw,
                                                theta=attn_kwargs.pop("rope_theta", 10000.0))
        if use_nan_mask_tokens:
            attn_kwargs["use_mask_token"] = True
        if self._is_rope and tokenizer == "patch_embed_2d":
            tokenizer_kwargs = dict(tokenizer_kwargs)
            asked = tokenizer_kwargs.get("pos_embed", None)
            if asked not in (None, "none"):
                warnings.warn("attention_backend='natten2d_rope' uses rotary position embeddings; overriding the requested "
                              f"pos_embed={asked!r} with 'none' to avoid double-counting the positional signal.",
                              UserWarning, stacklevel=2)
            tokenizer_kwargs["pos_embed"] = "none"
        if isinstance(tokenizer, str):
            if tokenizer not in ("patch_embed_2d", "hpx_patch_embed"):
                raise ValueError("tokenizer must be 'patch_embed_2d' or 'hpx_patch_embed'")
            self.tokenizer = get_tokenizer(input_size=self.input_size, patch_size=self.patch_size, in_channels=in_channels,
                                           hidden_size=hidden_size, tokenizer=tokenizer, **tokenizer_kwargs)
        elif isinstance(tokenizer, TokenizerModuleBase):
            self.tokenizer = tokenizer
        else:
            raise TypeError("tokenizer must be a string or a physicsnemo.core.Module instance subclassing physicsnemo.nn.TokenizerModuleBase")
        if isinstance(conditioning_embedder, str):
            self.conditioning_embedder = get_conditioning_embedder(
                ConditioningEmbedderType[conditioning_embedder.upper()], hidden_size=hidden_size,
                condition_dim=condition_dim or 0, amp_mode=self.meta.amp_gpu, **conditioning_embedder_kwargs)
        elif isinstance(conditioning_embedder, ConditioningEmbedder):
            self.conditioning_embedder = conditioning_embedder
        else:
            raise TypeError("conditioning_embedder must be a ConditioningEmbedderType or a Module implementing the ConditioningEmbedder protocol")
        if isinstance(detokenizer, str):
            if detokenizer not in ("proj_reshape_2d", "proj_reshape_2d_conv", "hpx_patch_detokenizer"):
                raise ValueError("detokenizer must be 'proj_reshape_2d', 'proj_reshape_2d_conv', or 'hpx_patch_detokenizer'")
            self.detokenizer = get_detokenizer(input_size=self.input_size, patch_size=self.patch_size,
                                               out_channels=self.out_channels, hidden_size=hidden_size,
                                               layernorm_backend=layernorm_backend, detokenizer=detokenizer, **detokenizer_kwargs)
        elif isinstance(detokenizer, DetokenizerModuleBase):
            self.detokenizer = detokenizer
        else:
            raise TypeError("detokenizer must be a string or a physicsnemo.core.Module instance subclassing physicsnemo.nn.DetokenizerModuleBase")
        if drop_path_rates is None:
            drop_path_rates = [0.0] * depth
        elif len(drop_path_rates) != depth:
            raise ValueError(f"drop_path_rates length ({len(drop_path_rates)}) must match DiT depth ({depth})")
        self.blocks = nn.ModuleList([
            DiTBlock(hidden_size, num_heads, attention_backend=attention_backend, layernorm_backend=layernorm_backend,
                     mlp_ratio=mlp_ratio, drop_path=drop_path_rates[i],
                     condition_embed_dim=self.conditioning_embedder.output_dim, **block_kwargs, **attn_kwargs)
            for i in range(depth)])
        if dit_initialization:
            self.initialize_weights()
        self.force_tokenization_fp32 = force_tokenization_fp32
        self.register_load_state_dict_pre_hook(self._migrate_legacy_checkpoint)

    @staticmethod
    def _migrate_legacy_checkpoint(module, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                   error_msgs):
        old, new = "t_embedder.", "conditioning_embedder.t_embedder."
        for key in [k for k in state_dict if k.startswith(old)]:
            target = new + key[len(old):]
            if key == old + "freqs":
                del state_dict[key]
            elif target not in state_dict:
                state_dict[target] = state_dict.pop(key)

    def initialize_weights(self):
        def basic(m):
            if isinstance(m, nn.Linear):
                torch.nn.init.xavier_uniform_(m.weight)
                if m.bias is not None:
                    nn.init.constant_(m.bias, 0)

        self.apply(basic)
        self.tokenizer.initialize_weights()
        self.detokenizer.initialize_weights()
        for b in self.blocks:
            b.initialize_weights()

    def _pixel_mask_to_token_mask(self, invalid_mask: torch.Tensor):
        nd = len(self.input_size)
        if invalid_mask.ndim == nd + 1:
            invalid_mask = invalid_mask.unsqueeze(1)
        if invalid_mask.ndim != nd + 2 or invalid_mask.shape[1] != 1:
            raise ValueError("invalid_mask must have shape (B, *spatial_dims) or (B, 1, *spatial_dims) matching the DiT "
                             f"spatial input; got shape {tuple(invalid_mask.shape)}")
        coarse = F.max_pool2d(invalid_mask.to(torch.float32), kernel_size=self.patch_size, stride=self.patch_size)
        return (coarse > 0).reshape(coarse.shape[0], -1)

    def _fp32(self, fn, x, *args, **kw):
        if not self.force_tokenization_fp32:
            return fn(x, *args, **kw)
        dt = x.dtype
        with torch.autocast(device_type="cuda", enabled=False):
            return fn(x.to(torch.float32), *args, **kw).to(dt)

    def forward(self, x, t, condition=None, p_dropout=None, attn_kwargs: Dict[str, Any] = {},
                tokenizer_kwargs: Dict[str, Any] = {}, invalid_mask=None):
        if invalid_mask is not None and not self._use_nan_mask_tokens:
            raise ValueError("invalid_mask was provided but the DiT was constructed with use_nan_mask_tokens=False, so no "
                             "learned mask tokens were allocated. Rebuild the model with use_nan_mask_tokens=True to use "
                             "dynamic invalid-region masking.")
        x = self._fp32(self.tokenizer, x, **tokenizer_kwargs)
        c = self.conditioning_embedder(t, condition=condition)
        kw = {**self.attn_kwargs_forward, **attn_kwargs}
        if self._is_rope:
            kw["rope_cos"], kw["rope_sin"] = self.rope(attn_kwargs.get("latent_hw"))
        if invalid_mask is not None:
            kw.setdefault("invalid_token_mask", self._pixel_mask_to_token_mask(invalid_mask))
        for blk in self.blocks:
            x = blk(x, c, p_dropout=p_dropout, attn_kwargs=kw)
        return self._fp32(self.detokenizer, x, c)
