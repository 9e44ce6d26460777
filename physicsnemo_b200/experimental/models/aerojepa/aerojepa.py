"""AeroJEPA: joint-embedding predictive model for aerodynamic fields on point clouds.

Parity: ``physicsnemo/experimental/models/aerojepa/trunk.py`` (``AeroJEPATrunk`` ``:40``) and
``aerojepa.py`` (``AeroJEPA`` ``:39``).  The trunk owns the geometry (context) encoder, the flow
(target) encoder and the field decoder; the model adds the predictor that maps geometry tokens to
flow tokens.  Training uses the pieces separately (encode both views, predict, decode); inference
(``forward``) needs geometry and operating conditions only: encode the geometry, place target tokens
with the target encoder's tokenizer, predict their features, decode at the query points.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ....core.module import Module
from ....nn.module.mlp_layers import Mlp
from .encoders import BaseContextEncoder, BaseTargetEncoder
from .predictor import PrototypeTokenJEPAHead
from .tokens import TokenSet


class AeroJEPATrunk(Module):
    """Context encoder + target encoder + decoder, with an optional fluid / solid mask head on the query embeddings."""

    def __init__(self, *, context_encoder: BaseContextEncoder, target_encoder: BaseTargetEncoder, decoder: Module,
                 include_geometry_global_in_decoder_cond: bool = True, mask_prediction_enabled: bool = False,
                 mask_head_hidden_dim: int = 128, mask_head_use_cond: bool = True):
        super().__init__()
        self.context_encoder, self.target_encoder, self.decoder = context_encoder, target_encoder, decoder
        self.include_geometry_global_in_decoder_cond = bool(include_geometry_global_in_decoder_cond)
        self.mask_prediction_enabled, self.mask_head_use_cond = bool(mask_prediction_enabled), bool(mask_head_use_cond)
        self.mask_head = None
        if self.mask_prediction_enabled:
            width = (int(decoder.query_in.out_features) + (int(getattr(decoder, "cond_dim", 0)) if self.mask_head_use_cond else 0)
                     + int(bool(getattr(decoder, "use_sdf", True))))
            self.mask_head = Mlp(in_features=width, hidden_features=[int(mask_head_hidden_dim)] * 2, out_features=1,
                                 act_layer=nn.SiLU, final_dropout=False)

    @staticmethod
    def supports_batched_forward() -> bool:
        return True

    def decoder_condition(self, gen_params: torch.Tensor, context_global: Optional[torch.Tensor]) -> torch.Tensor:
        """``(B, G [+ C])``: operating conditions, followed by the geometry's global token when configured."""
        cond = gen_params.reshape(1, -1) if gen_params.ndim == 1 else gen_params
        if self.include_geometry_global_in_decoder_cond and context_global is not None:
            cond = torch.cat([cond, context_global.reshape(cond.shape[0], -1)], dim=-1)
        return cond

    # kept under the reference's names
    def _build_cond_global_single(self, *, gen_params, context_global):
        return self.decoder_condition(gen_params, context_global)

    def _build_cond_global_batched(self, *, gen_params, context_global):
        return self.decoder_condition(gen_params, context_global)

    def _mask_logits(self, embeddings, cond, sdf):
        parts = [embeddings] + ([cond] if self.mask_head_use_cond else []) + ([sdf] if getattr(self.decoder, "use_sdf", True) else [])
        return self.mask_head(torch.cat(parts, dim=-1))

    def encode_context(self, *, context_pos, context_feat, target_surface_pos, target_surface_main_feat, target_volume_pos,
                       target_volume_feat, gen_params) -> dict:
        ctx = self.context_encoder(context_pos=context_pos, context_feat=context_feat)
        tgt = self.target_encoder(surface_pos=target_surface_pos, surface_main_feat=target_surface_main_feat,
                                  volume_pos=target_volume_pos, volume_feat=target_volume_feat)
        glob = ctx.global_token if ctx.global_token is not None else ctx.tokens.global_token
        return {"context_tokens": ctx.tokens, "target_tokens": tgt.tokens, "cond_global": self.decoder_condition(gen_params, glob)}

    def decode_queries(self, *, context: dict, query_pos, query_sdf, return_mask_logits: bool = False):
        cond = context["cond_global"].reshape(1, -1).expand(query_pos.shape[0], -1)
        pred, emb = self.decoder(query_pos=query_pos, query_sdf=query_sdf, target_tokens=context["target_tokens"], cond=cond)
        if self.mask_head is None or not return_mask_logits:
            return pred
        return pred, self._mask_logits(emb, cond, query_sdf)

    def forward_single(self, *, context_pos, context_feat, target_surface_pos, target_surface_main_feat, target_volume_pos,
                       target_volume_feat, query_pos, query_sdf, gen_params, return_mask_logits: bool = False):
        ctx = self.encode_context(context_pos=context_pos, context_feat=context_feat, target_surface_pos=target_surface_pos,
                                  target_surface_main_feat=target_surface_main_feat, target_volume_pos=target_volume_pos,
                                  target_volume_feat=target_volume_feat, gen_params=gen_params)
        return self.decode_queries(context=ctx, query_pos=query_pos, query_sdf=query_sdf, return_mask_logits=return_mask_logits)

    def forward_batch(self, *, context_pos, context_feat, context_pos_n, target_surface_pos, target_surface_main_feat,
                      target_surface_pos_n, target_volume_pos, target_volume_feat, target_volume_pos_n, query_pos, query_sdf,
                      query_pos_n, gen_params, return_mask_logits: bool = False):
        ctx = self.context_encoder.forward_batched(context_pos=context_pos, context_feat=context_feat, context_pos_n=context_pos_n)
        tgt = self.target_encoder.forward_batched(
            surface_pos=target_surface_pos, surface_main_feat=target_surface_main_feat, surface_pos_n=target_surface_pos_n,
            volume_pos=target_volume_pos, volume_feat=target_volume_feat, volume_pos_n=target_volume_pos_n)
        glob = ctx.global_token if ctx.global_token is not None else ctx.tokens.global_token
        cond = self.decoder_condition(gen_params, glob)
        pred, emb = self.decoder.forward_batched(query_pos=query_pos, query_sdf=query_sdf, query_counts=query_pos_n,
                                                 target_tokens=tgt.tokens, cond=cond)
        if self.mask_head is None or not return_mask_logits:
            return pred
        return pred, self._mask_logits(emb, cond[:, None, :].expand(-1, query_pos.shape[1], -1), query_sdf)

    def forward(self, **kw):
        return self.forward_batch(**kw) if "context_pos_n" in kw else self.forward_single(**kw)


class AeroJEPA(Module):
    """Trunk plus predictor.  ``forward(context_pos, context_feat, gen_params, query_pos, query_sdf=None, conditions=None)`` → ``(Nq, C)``."""

    def __init__(self, *, trunk: AeroJEPATrunk, predictor: PrototypeTokenJEPAHead):
        super().__init__()
        self.trunk, self.predictor = trunk, predictor

    context_encoder = property(lambda self: self.trunk.context_encoder)
    target_encoder = property(lambda self: self.trunk.target_encoder)
    decoder = property(lambda self: self.trunk.decoder)
    mask_head = property(lambda self: self.trunk.mask_head)
    mask_head_use_cond = property(lambda self: self.trunk.mask_head_use_cond)
    include_geometry_global_in_decoder_cond = property(lambda self: self.trunk.include_geometry_global_in_decoder_cond)

    def encode_geometry(self, *, context_pos, context_feat, gen_params):
        """Geometry tokens and the decoder-side condition vector ``(G [+ C],)``."""
        ctx = self.trunk.context_encoder(context_pos=context_pos, context_feat=context_feat)
        glob = ctx.global_token if ctx.global_token is not None else ctx.tokens.global_token
        return ctx.tokens, self.trunk.decoder_condition(gen_params, glob).squeeze(0)

    def encode_geometry_and_flow(self, **views) -> dict:
        return self.trunk.encode_context(**views)

    def predict_field_tokens(self, *, context_tokens: TokenSet, target_positions, conditions=None):
        return self.predictor(context_tokens=context_tokens, target_positions=target_positions, cond=conditions)

    def decode_field(self, *, target_tokens: TokenSet, cond_global, query_pos, query_sdf=None, return_mask_logits: bool = False):
        return self.trunk.decode_queries(context={"target_tokens": target_tokens, "cond_global": cond_global},
                                         query_pos=query_pos, query_sdf=query_sdf, return_mask_logits=return_mask_logits)

    @torch.no_grad()
    def decode_field_chunked(self, *, target_tokens: TokenSet, cond_global, query_pos, query_sdf, chunk_size: int,
                             precision: str = "fp32") -> torch.Tensor:
        """Decode a large query set chunk by chunk on the model's device; the result is fp32 on the host."""
        device = next(self.parameters()).device
        low = {"fp16": torch.float16, "bf16": torch.bfloat16}.get(precision)
        step, out = max(1, int(chunk_size)), []
        with torch.autocast(device_type=device.type, dtype=low or torch.float32, enabled=low is not None):
            for lo in range(0, query_pos.shape[0], step):
                piece = self.decode_field(target_tokens=target_tokens, cond_global=cond_global,
                                          query_pos=query_pos[lo:lo + step].to(device), query_sdf=query_sdf[lo:lo + step].to(device))
                out.append(piece.detach().float().cpu())
        return torch.cat(out)

    def build_target_token_coords(self, *, point_positions: torch.Tensor) -> torch.Tensor:
        """Where the target encoder would put its tokens for this cloud (its tokenizer run on zero features)."""
        base = getattr(self.trunk.target_encoder, "encoder", None)
        if base is None or not hasattr(base, "_tokenize_single"):
            raise ValueError("Target encoder does not expose the transformer tokenization path.")
        zeros = point_positions.new_zeros(point_positions.shape[0], base.feature_in.in_features)
        return base._tokenize_single(point_positions=point_positions, point_features=zeros)[0]

    def forward(self, *, context_pos, context_feat, gen_params, query_pos, query_sdf=None, conditions=None) -> torch.Tensor:
        if context_pos.ndim != 2 or context_feat.ndim != 2:
            raise ValueError(f"context_pos and context_feat must be rank 2; got {tuple(context_pos.shape)} and "
                             f"{tuple(context_feat.shape)}.")
        if context_pos.shape[0] != context_feat.shape[0]:
            raise ValueError(f"context_pos and context_feat must agree on the point count; got {context_pos.shape[0]} vs "
                             f"{context_feat.shape[0]}.")
        if query_sdf is None and getattr(self.decoder, "use_sdf", False):
            raise ValueError("query_sdf must be provided when the decoder has use_sdf=True.")
        tokens, cond_global = self.encode_geometry(context_pos=context_pos, context_feat=context_feat, gen_params=gen_params)
        coords = self.build_target_token_coords(point_positions=context_pos)
        if conditions is None:
            conditions = gen_params.reshape(1, -1) if gen_params.ndim == 1 else gen_params
        feats = self.predict_field_tokens(context_tokens=tokens, target_positions=coords, conditions=conditions)
        if feats.ndim == 3 and feats.shape[0] == 1:
            feats = feats[0]
        predicted = TokenSet(features=feats, coords=coords, mask=torch.ones(coords.shape[0], dtype=torch.bool, device=coords.device))
        return self.decode_field(target_tokens=predicted, cond_global=cond_global, query_pos=query_pos, query_sdf=query_sdf)

    @torch.no_grad()
    def predict(self, **inputs) -> torch.Tensor:
        return self.forward(**inputs)
