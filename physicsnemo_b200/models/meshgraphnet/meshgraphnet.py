"""MeshGraphNet: encode → ``processor_size`` × (edge block, node block) → decode.

Parity: ``physicsnemo/models/meshgraphnet/meshgraphnet.py`` — ``MeshGraphNet`` (``:54-271``) and
``MeshGraphNetProcessor`` (``:274-515``, activation-checkpoint segments with optional CPU
offload).  State-dict keys: ``edge_encoder.model.*``, ``node_encoder.model.*``,
``processor.processor_layers.{2i}.edge_mlp.model.*``, ``processor.processor_layers.{2i+1}.node_mlp.model.*``,
``node_decoder.model.*``.  ``graph`` is any object with ``edge_index`` (2, E).
"""
from __future__ import annotations

from contextlib import nullcontext
from dataclasses import dataclass
from typing import Callable, Literal, Tuple
from warnings import warn

import torch
import torch.nn as nn
from torch import Tensor

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import get_activation
from ...nn.module.gnn_layers.mesh_edge_block import MeshEdgeBlock
from ...nn.module.gnn_layers.mesh_graph_mlp import MeshGraphMLP
from ...nn.module.gnn_layers.mesh_node_block import MeshNodeBlock
from ...nn.module.gnn_layers.utils import set_checkpoint_fn


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp_cpu: bool = False
    amp_gpu: bool = True
    torch_fx: bool = False
    bf16: bool = True
    onnx: bool = False
    func_torch: bool = True
    auto_grad: bool = True


def _expect_rows(what: str, t: Tensor, width: int) -> None:
    """``t`` must be a 2-D feature table with ``width`` columns."""
    if torch.compiler.is_compiling():
        return
    if t.ndim != 2 or t.shape[1] != width:
        raise ValueError(f"Expected tensor of shape (N_{what}, {width}) but got tensor of shape {tuple(t.shape)}")


class MeshGraphNetProcessor(nn.Module):
    """``processor_size`` message-passing steps, each an edge block followed by a node block.

    The ``2 · processor_size`` layers can be cut into equal activation-checkpoint segments
    (``num_processor_checkpoint_segments``), whose saved tensors may additionally be kept in pinned host memory
    (``checkpoint_offloading``).
    """

    def __init__(self, processor_size: int = 15, input_dim_node: int = 128, input_dim_edge: int = 128,
                 num_layers_node: int = 2, num_layers_edge: int = 2, aggregation: str = "sum",
                 norm_type: str = "LayerNorm", activation_fn: nn.Module = nn.ReLU(), do_concat_trick: bool = False,
                 num_processor_checkpoint_segments: int = 0, checkpoint_offloading: bool = False):
        super().__init__()
        self.processor_size, self.input_dim_node, self.input_dim_edge = processor_size, input_dim_node, input_dim_edge
        self.num_processor_checkpoint_segments = num_processor_checkpoint_segments
        self.checkpoint_offloading = bool(checkpoint_offloading) and num_processor_checkpoint_segments > 0
        width = input_dim_edge
        layers = []
        for _ in range(processor_size):
            layers.append(MeshEdgeBlock(input_dim_node, width, width, width, num_layers_edge, activation_fn, norm_type,
                                        do_concat_trick, False))
            layers.append(MeshNodeBlock(aggregation, input_dim_node, width, width, width, num_layers_node, activation_fn,
                                        norm_type, False))
        self.processor_layers = nn.ModuleList(layers)
        self.num_processor_layers = 2 * processor_size
        self.set_checkpoint_segments(num_processor_checkpoint_segments)
        self.set_checkpoint_offload_ctx(self.checkpoint_offloading)

    def set_checkpoint_offload_ctx(self, enabled: bool) -> None:
        """Keep the tensors saved inside checkpointed segments on the host (pinned) when ``enabled``."""
        self.checkpoint_offload_ctx = torch.autograd.graph.save_on_cpu(pin_memory=True) if enabled else nullcontext()

    def set_checkpoint_segments(self, checkpoint_segments: int) -> None:
        """Cut the layer list into ``checkpoint_segments`` equal parts (0: one part, no recomputation)."""
        n = self.num_processor_layers
        if checkpoint_segments > 0 and n % checkpoint_segments:
            raise ValueError("Processor layers must be a multiple of checkpoint_segments")
        per_part = n // checkpoint_segments if checkpoint_segments > 0 else n
        self.checkpoint_segments = [(lo, lo + per_part) for lo in range(0, n, max(per_part, 1))] or [(0, 0)]
        self.checkpoint_fn = set_checkpoint_fn(checkpoint_segments > 0)

    _set_checkpoint_segments = set_checkpoint_segments
    _set_checkpoint_offload_ctx = set_checkpoint_offload_ctx

    def run_function(self, segment_start: int, segment_end: int) -> Callable:
        """Callable ``(nodes, edges, graph) → (edges, nodes)`` that applies layers ``[segment_start, segment_end)``."""
        part = list(self.processor_layers[segment_start:segment_end])

        def apply(nodes: Tensor, edges: Tensor, graph) -> Tuple[Tensor, Tensor]:
            for layer in part:
                edges, nodes = layer(edges, nodes, graph)
            return edges, nodes

        return apply

    def forward(self, node_features: Tensor, edge_features: Tensor, graph) -> Tensor:
        _expect_rows("nodes", node_features, self.input_dim_node)
        _expect_rows("edges", edge_features, self.input_dim_edge)
        nodes, edges = node_features, edge_features
        with self.checkpoint_offload_ctx:
            for lo, hi in self.checkpoint_segments:
                edges, nodes = self.checkpoint_fn(self.run_function(lo, hi), nodes, edges, graph, use_reentrant=False,
                                                  preserve_rng_state=False)
        return nodes


class MeshGraphNet(Module):
    """MeshGraphNet; ``forward(node_features (N, Dn), edge_features (E, De), graph) -> (N, Dout)``."""

    def __init__(self, input_dim_nodes: int, input_dim_edges: int, output_dim: int, processor_size: int = 15,
                 mlp_activation_fn: str = "relu", num_layers_node_processor: int = 2,
                 num_layers_edge_processor: int = 2, hidden_dim_processor: int = 128,
                 hidden_dim_node_encoder: int = 128, num_layers_node_encoder: int = 2,
                 hidden_dim_edge_encoder: int = 128, num_layers_edge_encoder: int = 2,
                 hidden_dim_node_decoder: int = 128, num_layers_node_decoder: int = 2,
                 aggregation: Literal["sum", "mean"] = "sum", do_concat_trick: bool = False,
                 num_processor_checkpoint_segments: int = 0, checkpoint_offloading: bool = False,
                 recompute_activation: bool = False, norm_type: Literal["LayerNorm", "TELayerNorm"] = "LayerNorm"):
        super().__init__(meta=MetaData())
        depth = {"num_layers_node_encoder": num_layers_node_encoder, "num_layers_edge_encoder": num_layers_edge_encoder,
                 "num_layers_node_decoder": num_layers_node_decoder}
        for name, value in depth.items():
            if value is None:
                raise ValueError(f"{name} cannot be None")
        if norm_type not in ("LayerNorm", "TELayerNorm"):
            raise ValueError("Norm type should be either 'LayerNorm' or 'TELayerNorm'")
        if norm_type == "TELayerNorm" and not torch.cuda.is_available():
            warn("TELayerNorm is not supported on CPU. Switching to LayerNorm.")
            norm_type = "LayerNorm"
        self.input_dim_nodes, self.input_dim_edges, self.output_dim = input_dim_nodes, input_dim_edges, output_dim
        act = get_activation(mlp_activation_fn)
        latent = hidden_dim_processor

        def mlp(n_in: int, n_out: int, hidden: int, layers: int, norm) -> MeshGraphMLP:
            return MeshGraphMLP(n_in, output_dim=n_out, hidden_dim=hidden, hidden_layers=layers, activation_fn=act,
                                norm_type=norm, recompute_activation=recompute_activation)

        self.edge_encoder = mlp(input_dim_edges, latent, hidden_dim_edge_encoder, num_layers_edge_encoder, norm_type)
        self.node_encoder = mlp(input_dim_nodes, latent, hidden_dim_node_encoder, num_layers_node_encoder, norm_type)
        self.node_decoder = mlp(latent, output_dim, hidden_dim_node_decoder, num_layers_node_decoder, None)
        self.processor = MeshGraphNetProcessor(
            processor_size=processor_size, input_dim_node=latent, input_dim_edge=latent, num_layers_node=num_layers_node_processor,
            num_layers_edge=num_layers_edge_processor, aggregation=aggregation, norm_type=norm_type, activation_fn=act,
            do_concat_trick=do_concat_trick, num_processor_checkpoint_segments=num_processor_checkpoint_segments,
            checkpoint_offloading=checkpoint_offloading)

    def forward(self, node_features: Tensor, edge_features: Tensor, graph, **kwargs) -> Tensor:
        _expect_rows("nodes", node_features, self.input_dim_nodes)
        _expect_rows("edges", edge_features, self.input_dim_edges)
        latent_nodes = self.processor(self.node_encoder(node_features), self.edge_encoder(edge_features), graph)
        return self.node_decoder(latent_nodes)
