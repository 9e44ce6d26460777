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
from itertools import chain
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


class MeshGraphNetProcessor(nn.Module):
    """Alternating edge / node blocks with optional activation-checkpoint segments."""

    def __init__(self, processor_size: int = 15, input_dim_node: int = 128, input_dim_edge: int = 128,
                 num_layers_node: int = 2, num_layers_edge: int = 2, aggregation: str = "sum",
                 norm_type: str = "LayerNorm", activation_fn: nn.Module = nn.ReLU(), do_concat_trick: bool = False,
                 num_processor_checkpoint_segments: int = 0, checkpoint_offloading: bool = False):
        super().__init__()
        self.processor_size = processor_size
        self.num_processor_checkpoint_segments = num_processor_checkpoint_segments
        self.input_dim_node, self.input_dim_edge = input_dim_node, input_dim_edge
        self.checkpoint_offloading = checkpoint_offloading if num_processor_checkpoint_segments > 0 else False
        edge_blocks = [MeshEdgeBlock(input_dim_node, input_dim_edge, input_dim_edge, input_dim_edge, num_layers_edge,
                                     activation_fn, norm_type, do_concat_trick, False) for _ in range(processor_size)]
        node_blocks = [MeshNodeBlock(aggregation, input_dim_node, input_dim_edge, input_dim_edge, input_dim_edge,
                                     num_layers_node, activation_fn, norm_type, False) for _ in range(processor_size)]
        self.processor_layers = nn.ModuleList(list(chain(*zip(edge_blocks, node_blocks))))
        self.num_processor_layers = len(self.processor_layers)
        self.set_checkpoint_segments(num_processor_checkpoint_segments)
        self.set_checkpoint_offload_ctx(self.checkpoint_offloading)

    def set_checkpoint_offload_ctx(self, enabled: bool) -> None:
        self.checkpoint_offload_ctx = torch.autograd.graph.save_on_cpu(pin_memory=True) if enabled else nullcontext()

    def set_checkpoint_segments(self, checkpoint_segments: int) -> None:
        if checkpoint_segments > 0:
            if self.num_processor_layers % checkpoint_segments != 0:
                raise ValueError("Processor layers must be a multiple of checkpoint_segments")
            size = self.num_processor_layers // checkpoint_segments
            self.checkpoint_segments = [(i, i + size) for i in range(0, self.num_processor_layers, size)]
            self.checkpoint_fn = set_checkpoint_fn(True)
        else:
            self.checkpoint_fn = set_checkpoint_fn(False)
            self.checkpoint_segments = [(0, self.num_processor_layers)]

    _set_checkpoint_segments = set_checkpoint_segments
    _set_checkpoint_offload_ctx = set_checkpoint_offload_ctx

    def run_function(self, segment_start: int, segment_end: int) -> Callable:
        segment = self.processor_layers[segment_start:segment_end]

        def custom_forward(node_features: Tensor, edge_features: Tensor, graph) -> Tuple[Tensor, Tensor]:
            for module in segment:
                edge_features, node_features = module(edge_features, node_features, graph)
            return edge_features, node_features

        return custom_forward

    def forward(self, node_features: Tensor, edge_features: Tensor, graph) -> Tensor:
        if not torch.compiler.is_compiling():
            if node_features.ndim != 2 or node_features.shape[1] != self.input_dim_node:
                raise ValueError(
                    f"Expected tensor of shape (N_nodes, {self.input_dim_node}) but got tensor of shape {tuple(node_features.shape)}"
                )
            if edge_features.ndim != 2 or edge_features.shape[1] != self.input_dim_edge:
                raise ValueError(
                    f"Expected tensor of shape (N_edges, {self.input_dim_edge}) but got tensor of shape {tuple(edge_features.shape)}"
                )
        with self.checkpoint_offload_ctx:
            for start, end in self.checkpoint_segments:
                edge_features, node_features = self.checkpoint_fn(
                    self.run_function(start, end), node_features, edge_features, graph,
                    use_reentrant=False, preserve_rng_state=False)
        return node_features


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
        self.input_dim_nodes, self.input_dim_edges, self.output_dim = input_dim_nodes, input_dim_edges, output_dim
        activation_fn = get_activation(mlp_activation_fn)
        if num_layers_node_encoder is None:
            raise ValueError("num_layers_node_encoder cannot be None")
        if num_layers_edge_encoder is None:
            raise ValueError("num_layers_edge_encoder cannot be None")
        if num_layers_node_decoder is None:
            raise ValueError("num_layers_node_decoder cannot be None")
        if norm_type not in ["LayerNorm", "TELayerNorm"]:
            raise ValueError("Norm type should be either 'LayerNorm' or 'TELayerNorm'")
        if not torch.cuda.is_available() and norm_type == "TELayerNorm":
            warn("TELayerNorm is not supported on CPU. Switching to LayerNorm.")
            norm_type = "LayerNorm"
        self.edge_encoder = MeshGraphMLP(input_dim_edges, output_dim=hidden_dim_processor,
                                         hidden_dim=hidden_dim_edge_encoder, hidden_layers=num_layers_edge_encoder,
                                         activation_fn=activation_fn, norm_type=norm_type,
                                         recompute_activation=recompute_activation)
        self.node_encoder = MeshGraphMLP(input_dim_nodes, output_dim=hidden_dim_processor,
                                         hidden_dim=hidden_dim_node_encoder, hidden_layers=num_layers_node_encoder,
                                         activation_fn=activation_fn, norm_type=norm_type,
                                         recompute_activation=recompute_activation)
        self.node_decoder = MeshGraphMLP(hidden_dim_processor, output_dim=output_dim,
                                         hidden_dim=hidden_dim_node_decoder, hidden_layers=num_layers_node_decoder,
                                         activation_fn=activation_fn, norm_type=None,
                                         recompute_activation=recompute_activation)
        self.processor = MeshGraphNetProcessor(
            processor_size=processor_size, input_dim_node=hidden_dim_processor, input_dim_edge=hidden_dim_processor,
            num_layers_node=num_layers_node_processor, num_layers_edge=num_layers_edge_processor,
            aggregation=aggregation, norm_type=norm_type, activation_fn=activation_fn,
            do_concat_trick=do_concat_trick, num_processor_checkpoint_segments=num_processor_checkpoint_segments,
            checkpoint_offloading=checkpoint_offloading)

    def forward(self, node_features: Tensor, edge_features: Tensor, graph, **kwargs) -> Tensor:
        if not torch.compiler.is_compiling():
            if node_features.ndim != 2 or node_features.shape[1] != self.input_dim_nodes:
                raise ValueError(
                    f"Expected tensor of shape (N_nodes, {self.input_dim_nodes}) but got tensor of shape {tuple(node_features.shape)}"
                )
            if edge_features.ndim != 2 or edge_features.shape[1] != self.input_dim_edges:
                raise ValueError(
                    f"Expected tensor of shape (N_edges, {self.input_dim_edges}) but got tensor of shape {tuple(edge_features.shape)}"
                )
        edge_features = self.edge_encoder(edge_features)
        node_features = self.node_encoder(node_features)
        x = self.processor(node_features, edge_features, graph)
        return self.node_decoder(x)
