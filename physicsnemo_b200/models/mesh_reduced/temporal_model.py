"""Causal transformer over latent sequences of the mesh-reduced model.

Parity: ``physicsnemo/models/mesh_reduced/temporal_model.py`` (``Sequence_Model``: context / input /
output ``MeshGraphMLP`` encoders around a decoder-only transformer with a causal mask; ``sample``
rolls the model out auto-regressively).  ``dist`` only supplies the device of the mask; any object
with a ``device`` attribute (or ``None``: the input's device) works.
"""
from __future__ import annotations

import torch
from torch import Tensor, nn
from torch.nn import LayerNorm

from ...nn.module.gnn_layers.mesh_graph_mlp import MeshGraphMLP
from ...nn.module.transformer_decoder import DecoderOnlyLayer, TransformerDecoder


class Sequence_Model(torch.nn.Module):
    def __init__(self, input_dim: int, input_context_dim: int, dist, dropout_rate: float = 0.0, num_layers_decoder: int = 3,
                 num_heads: int = 8, dim_feedforward_scale: int = 4, num_layers_context_encoder: int = 2,
                 num_layers_input_encoder: int = 2, num_layers_output_encoder: int = 2, activation: str = "gelu"):
        super().__init__()
        self.dist = dist
        layer = DecoderOnlyLayer(input_dim, num_heads, dim_feedforward_scale * input_dim, dropout_rate, activation,
                                 layer_norm_eps=1e-5, batch_first=True, norm_first=False, bias=True)
        self.decoder = TransformerDecoder(layer, num_layers_decoder, LayerNorm(input_dim, eps=1e-5, bias=True))
        self.input_dim, self.input_context_dim = input_dim, input_context_dim

        def mlp(inp, layers, norm):
            return MeshGraphMLP(inp, output_dim=input_dim, hidden_dim=input_dim * 2, hidden_layers=layers,
                                activation_fn=nn.ReLU(), norm_type=norm, recompute_activation=False)

        self.input_encoder = mlp(input_dim, num_layers_input_encoder, "LayerNorm")
        self.output_encoder = mlp(input_dim, num_layers_output_encoder, None)
        self.context_encoder = mlp(input_context_dim, num_layers_context_encoder, "LayerNorm")

    def forward(self, x: Tensor, context: Tensor | None = None) -> Tensor:
        if not torch.compiler.is_compiling():
            if x.ndim != 3 or x.shape[-1] != self.input_dim:
                raise ValueError(f"Expected tensor of shape (B, T, {self.input_dim}) but got tensor of shape {tuple(x.shape)}")
            if context is not None and (context.ndim != 3 or context.shape[-1] != self.input_context_dim):
                raise ValueError(f"Expected context shape (B, T_c, {self.input_context_dim}) but got tensor of shape {tuple(context.shape)}")
        if context is not None:
            x = torch.cat([self.context_encoder(context), x], dim=1)
        x = self.input_encoder(x)
        device = getattr(self.dist, "device", None) or x.device
        mask = self.generate_square_subsequent_mask(x.size(1), device=device, dtype=x.dtype)
        return self.output_encoder(self.decoder(x, tgt_mask=mask))[:, 1:]

    @torch.no_grad()
    def sample(self, z0: Tensor, step_size: int, context: Tensor | None = None):
        z = z0
        for _ in range(step_size):
            z = torch.concat([z, self.forward(z, context)[:, -1].unsqueeze(1)], dim=1)
        return z

    @staticmethod
    def generate_square_subsequent_mask(sz: int, device=None, dtype: torch.dtype | None = None) -> Tensor:
        dtype = dtype or torch.get_default_dtype()
        return torch.triu(torch.full((sz, sz), float("-inf"), dtype=dtype, device=device), diagonal=1)
