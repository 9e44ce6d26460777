"""Processors of GraphCast: message passing on the multimesh, or masked self-attention over mesh nodes.

Parity: ``physicsnemo/models/graphcast/graph_cast_processor.py`` (``GraphCastProcessor``:
alternating ``MeshEdgeBlock`` / ``MeshNodeBlock`` with activation-checkpoint segments;
``GraphCastProcessorGraphTransformer``: a stack of pre-norm transformer layers with a k-hop
attention mask).  The reference builds the transformer variant from Transformer-Engine layers and
cannot construct it without that package; here it is built from this package's own layers
(``nn.MultiheadAttention``-free: fused QKV ``Linear``, SDPA with the boolean mask, GELU MLP), so
its parameter names are this package's, not Transformer-Engine's.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ...nn.module.gnn_layers.mesh_edge_block import MeshEdgeBlock
from ...nn.module.gnn_layers.mesh_node_block import MeshNodeBlock
from ...nn.module.gnn_layers.utils import set_checkpoint_fn


class GraphCastProcessor(nn.Module):
    def __init__(self, aggregation: str = "sum", processor_layers: int = 16, input_dim_nodes: int = 512,
                 input_dim_edges: int = 512, hidden_dim: int = 512, hidden_layers: int = 1,
                 activation_fn: nn.Module = nn.SiLU(), norm_type: str = "LayerNorm", do_concat_trick: bool = False,
                 recompute_activation: bool = False):
        super().__init__()
        layers = []
        for _ in range(processor_layers):
            layers.append(MeshEdgeBlock(input_dim_nodes, input_dim_edges, input_dim_edges, hidden_dim, hidden_layers,
                                        activation_fn, norm_type, do_concat_trick, recompute_activation))
            layers.append(MeshNodeBlock(aggregation, input_dim_nodes, input_dim_edges, input_dim_nodes, hidden_dim,
                                        hidden_layers, activation_fn, norm_type, recompute_activation))
        self.processor_layers = nn.ModuleList(layers)
        self.num_processor_layers = len(self.processor_layers)
        self.set_checkpoint_segments(0)

    def set_checkpoint_segments(self, checkpoint_segments: int) -> None:
        n = self.num_processor_layers
        if checkpoint_segments > 0:
            if n % checkpoint_segments != 0:
                raise ValueError("Processor layers must be a multiple of checkpoint_segments")
            size = n // checkpoint_segments
            self.checkpoint_segments = [(i, i + size) for i in range(0, n, size)]
            self.checkpoint_fn = set_checkpoint_fn(True)
        else:
            self.checkpoint_segments = [(0, n)]
            self.checkpoint_fn = set_checkpoint_fn(False)

    def run_function(self, segment_start: int, segment_end: int):
        segment = self.processor_layers[segment_start:segment_end]

        def custom_forward(efeat, nfeat, graph):
            for module in segment:
                efeat, nfeat = module(efeat, nfeat, graph)
            return efeat, nfeat

        return custom_forward

    def forward(self, efeat: Tensor, nfeat: Tensor, graph):
        for start, end in self.checkpoint_segments:
            efeat, nfeat = self.checkpoint_fn(self.run_function(start, end), efeat, nfeat, graph, use_reentrant=False,
                                              preserve_rng_state=False)
        return efeat, nfeat


class _MaskedTransformerLayer(nn.Module):
    def __init__(self, hidden_size: int, ffn_hidden_size: int, num_heads: int):
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError("hidden size must be divisible by the number of attention heads")
        self.num_heads = num_heads
        self.ln_attn = nn.LayerNorm(hidden_size)
        self.qkv = nn.Linear(hidden_size, 3 * hidden_size)
        self.proj = nn.Linear(hidden_size, hidden_size)
        self.ln_mlp = nn.LayerNorm(hidden_size)
        self.fc1 = nn.Linear(hidden_size, ffn_hidden_size)
        self.fc2 = nn.Linear(ffn_hidden_size, hidden_size)

    def forward(self, x: Tensor, allowed: Tensor) -> Tensor:           # x [N, C]; allowed [N, N] True = may attend
        n, c = x.shape
        q, k, v = self.qkv(self.ln_attn(x)).reshape(n, 3, self.num_heads, c // self.num_heads).permute(1, 2, 0, 3)
        a = F.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=allowed)[0]
        x = x + self.proj(a.permute(1, 0, 2).reshape(n, c))
        return x + self.fc2(F.gelu(self.fc1(self.ln_mlp(x))))


class GraphCastProcessorGraphTransformer(nn.Module):
    """Self-attention over the mesh nodes restricted to k-hop neighbourhoods (``attention_mask``: True = blocked)."""

    def __init__(self, attention_mask: Tensor, num_attention_heads: int = 4, processor_layers: int = 16,
                 input_dim_nodes: int = 512, hidden_dim: int = 512):
        super().__init__()
        self.num_attention_heads = num_attention_heads
        self.hidden_dim = hidden_dim
        mask = torch.as_tensor(attention_mask, dtype=torch.bool)
        allowed = ~mask
        allowed |= torch.eye(mask.shape[0], dtype=torch.bool)            # a node always sees itself
        self.register_buffer("mask", mask, persistent=False)
        self.register_buffer("allowed", allowed, persistent=False)
        self.processor_layers = nn.ModuleList(
            [_MaskedTransformerLayer(input_dim_nodes, hidden_dim, num_attention_heads) for _ in range(processor_layers)])

    def forward(self, nfeat: Tensor) -> Tensor:
        for layer in self.processor_layers:
            nfeat = layer(nfeat, self.allowed)
        return nfeat
