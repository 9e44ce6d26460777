"""MeshGraphNet variants: KAN node encoder, bi-stride multi-scale processor, mesh + world edge sets.

Parity: ``physicsnemo/models/meshgraphnet/meshgraphkan.py`` (``MeshGraphKAN``: node encoder replaced by a
``KolmogorovArnoldNetwork``), ``bsms_mgn.py`` (``BiStrideMeshGraphNet``: the standard processor
followed by ``bistride_unet_levels`` passes of ``BistrideGraphMessagePassing`` over precomputed
multi-scale edge lists ``ms_edges`` and kept-node ids ``ms_ids``; node positions from ``graph.pos``),
``hybrid_meshgraphnet.py`` (``HybridMeshGraphNet`` / ``HybridMeshGraphNetProcessor``: separate encoders
and edge MLPs for mesh and world edges, joint aggregation).
"""
from __future__ import annotations

from dataclasses import dataclass
from itertools import chain
from typing import Callable, Iterable, Literal, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch import Tensor

from ...core.meta import ModelMetaData
from ...nn.module.activations import get_activation
from ...nn.module.gnn_layers.bsms import BistrideGraphMessagePassing
from ...nn.module.gnn_layers.mesh_edge_block import HybridMeshEdgeBlock
from ...nn.module.gnn_layers.mesh_graph_mlp import MeshGraphMLP
from ...nn.module.gnn_layers.mesh_node_block import HybridMeshNodeBlock
from ...nn.module.kan_layers import KolmogorovArnoldNetwork
from .meshgraphnet import MeshGraphNet, MeshGraphNetProcessor


@dataclass
class _VariantMetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp_cpu: bool = False
    amp_gpu: bool = True
    torch_fx: bool = False
    onnx: bool = False
    func_torch: bool = True
    auto_grad: bool = True


def _check(t: Tensor, width: int, what: str) -> None:
    if not torch.compiler.is_compiling() and (t.ndim != 2 or t.shape[1] != width):
        raise ValueError(f"Expected tensor of shape ({what}, {width}) but got tensor of shape {tuple(t.shape)}")


class MeshGraphKAN(MeshGraphNet):
    def __init__(self, input_dim_nodes: int, input_dim_edges: int, output_dim: int, processor_size: int = 15,
                 mlp_activation_fn: str = "relu", num_layers_node_processor: int = 2, num_layers_edge_processor: int = 2,
                 hidden_dim_processor: int = 128, hidden_dim_node_encoder: int = 128,
                 num_layers_node_encoder: Union[int, None] = 2, hidden_dim_edge_encoder: int = 128,
                 num_layers_edge_encoder: Union[int, None] = 2, hidden_dim_node_decoder: int = 128,
                 num_layers_node_decoder: Union[int, None] = 2, aggregation: Literal["sum", "mean"] = "sum",
                 do_concat_trick: bool = False, num_processor_checkpoint_segments: int = 0,
                 checkpoint_offloading: bool = False, recompute_activation: bool = False, num_harmonics: int = 5):
        super().__init__(input_dim_nodes=input_dim_nodes, input_dim_edges=input_dim_edges, output_dim=output_dim,
                         processor_size=processor_size, mlp_activation_fn=mlp_activation_fn,
                         num_layers_node_processor=num_layers_node_processor,
                         num_layers_edge_processor=num_layers_edge_processor, hidden_dim_processor=hidden_dim_processor,
                         hidden_dim_node_encoder=hidden_dim_node_encoder, num_layers_node_encoder=num_layers_node_encoder,
                         hidden_dim_edge_encoder=hidden_dim_edge_encoder, num_layers_edge_encoder=num_layers_edge_encoder,
                         hidden_dim_node_decoder=hidden_dim_node_decoder, num_layers_node_decoder=num_layers_node_decoder,
                         aggregation=aggregation, do_concat_trick=do_concat_trick,
                         num_processor_checkpoint_segments=num_processor_checkpoint_segments,
                         checkpoint_offloading=checkpoint_offloading, recompute_activation=recompute_activation,
                         norm_type="LayerNorm")
        self.meta = _VariantMetaData()
        self.node_encoder = KolmogorovArnoldNetwork(input_dim=input_dim_nodes, output_dim=hidden_dim_processor,
                                                    num_harmonics=num_harmonics, add_bias=True)


class BiStrideMeshGraphNet(MeshGraphNet):
    def __init__(self, input_dim_nodes: int, input_dim_edges: int, output_dim: int, processor_size: int = 15,
                 mlp_activation_fn: str = "relu", num_layers_node_processor: int = 2, num_layers_edge_processor: int = 2,
                 num_mesh_levels: int = 2, bistride_pos_dim: int = 3, num_layers_bistride: int = 2,
                 bistride_unet_levels: int = 1, hidden_dim_processor: int = 128, hidden_dim_node_encoder: int = 128,
                 num_layers_node_encoder: Optional[int] = 2, hidden_dim_edge_encoder: int = 128,
                 num_layers_edge_encoder: Optional[int] = 2, hidden_dim_node_decoder: int = 128,
                 num_layers_node_decoder: Optional[int] = 2, aggregation: Literal["sum", "mean"] = "sum",
                 do_concat_trick: bool = False, num_processor_checkpoint_segments: int = 0,
                 recompute_activation: bool = False):
        super().__init__(input_dim_nodes, input_dim_edges, output_dim, processor_size=processor_size,
                         mlp_activation_fn=mlp_activation_fn, num_layers_node_processor=num_layers_node_processor,
                         num_layers_edge_processor=num_layers_edge_processor, hidden_dim_processor=hidden_dim_processor,
                         hidden_dim_node_encoder=hidden_dim_node_encoder, num_layers_node_encoder=num_layers_node_encoder,
                         hidden_dim_edge_encoder=hidden_dim_edge_encoder, num_layers_edge_encoder=num_layers_edge_encoder,
                         hidden_dim_node_decoder=hidden_dim_node_decoder, num_layers_node_decoder=num_layers_node_decoder,
                         aggregation=aggregation, do_concat_trick=do_concat_trick,
                         num_processor_checkpoint_segments=num_processor_checkpoint_segments,
                         recompute_activation=recompute_activation)
        self.meta = _VariantMetaData()
        self.bistride_unet_levels = bistride_unet_levels
        self.bistride_processor = BistrideGraphMessagePassing(unet_depth=num_mesh_levels, latent_dim=hidden_dim_processor,
                                                              hidden_layer=num_layers_bistride, pos_dim=bistride_pos_dim)

    def forward(self, node_features: Tensor, edge_features: Tensor, graph, ms_edges: Iterable[Tensor] = (),
                ms_ids: Iterable[Tensor] = (), **kwargs) -> Tensor:
        _check(node_features, self.input_dim_nodes, "N_nodes")
        _check(edge_features, self.input_dim_edges, "N_edges")
        x = self.processor(self.node_encoder(node_features), self.edge_encoder(edge_features), graph)
        pos = graph.pos
        ms_edges = [e.to(pos.device).squeeze(0) if e.dim() == 3 else e.to(pos.device) for e in ms_edges]
        ms_ids = [i.squeeze(0) if i.dim() == 2 else i for i in ms_ids]
        for _ in range(self.bistride_unet_levels):
            x = self.bistride_processor(x, ms_ids, ms_edges, pos)
        return self.node_decoder(x)


class HybridMeshGraphNetProcessor(MeshGraphNetProcessor):
    def __init__(self, processor_size: int = 15, input_dim_node: int = 128, input_dim_edge: int = 128,
                 num_layers_node: int = 2, num_layers_edge: int = 2, aggregation: Literal["sum", "mean"] = "sum",
                 norm_type: Literal["LayerNorm", "TELayerNorm"] = "LayerNorm", activation_fn: nn.Module = nn.ReLU(),
                 do_concat_trick: bool = False, num_processor_checkpoint_segments: int = 0,
                 checkpoint_offloading: bool = False):
        super().__init__(processor_size=processor_size, input_dim_node=input_dim_node, input_dim_edge=input_dim_edge,
                         num_layers_node=num_layers_node, num_layers_edge=num_layers_edge, aggregation=aggregation,
                         norm_type=norm_type, activation_fn=activation_fn, do_concat_trick=do_concat_trick,
                         num_processor_checkpoint_segments=num_processor_checkpoint_segments,
                         checkpoint_offloading=checkpoint_offloading)
        edge_blocks = [HybridMeshEdgeBlock(input_dim_node, input_dim_edge, input_dim_edge, input_dim_edge, num_layers_edge,
                                           activation_fn, norm_type, do_concat_trick, False) for _ in range(processor_size)]
        node_blocks = [HybridMeshNodeBlock(aggregation, input_dim_node, input_dim_edge, input_dim_edge, input_dim_edge,
                                           num_layers_node, activation_fn, norm_type, False) for _ in range(processor_size)]
        self.processor_layers = nn.ModuleList(list(chain(*zip(edge_blocks, node_blocks))))
        self.num_processor_layers = len(self.processor_layers)
        self.set_checkpoint_segments(num_processor_checkpoint_segments)

    def _run_function(self, segment_start: int, segment_end: int) -> Callable:
        segment = self.processor_layers[segment_start:segment_end]

        def _custom_forward(node_features, mesh_edge_features, world_edge_features, graph) -> Tuple[Tensor, Tensor, Tensor]:
            for module in segment:
                mesh_edge_features, world_edge_features, node_features = module(mesh_edge_features, world_edge_features,
                                                                                node_features, graph)
            return mesh_edge_features, world_edge_features, node_features

        return _custom_forward

    def forward(self, node_features: Tensor, mesh_edge_features: Tensor, world_edge_features: Tensor, graph) -> Tensor:
        _check(node_features, self.input_dim_node, "N_nodes")
        _check(mesh_edge_features, self.input_dim_edge, "N_mesh_edges")
        _check(world_edge_features, self.input_dim_edge, "N_world_edges")
        with self.checkpoint_offload_ctx:
            for start, end in self.checkpoint_segments:
                mesh_edge_features, world_edge_features, node_features = self.checkpoint_fn(
                    self._run_function(start, end), node_features, mesh_edge_features, world_edge_features, graph,
                    use_reentrant=False, preserve_rng_state=False)
        return node_features


class HybridMeshGraphNet(MeshGraphNet):
    def __init__(self, input_dim_nodes: int, input_dim_edges: int, output_dim: int, processor_size: int = 15,
                 mlp_activation_fn: str = "relu", num_layers_node_processor: int = 2, num_layers_edge_processor: int = 2,
                 hidden_dim_processor: int = 128, hidden_dim_node_encoder: int = 128,
                 num_layers_node_encoder: Union[int, None] = 2, hidden_dim_edge_encoder: int = 128,
                 num_layers_edge_encoder: Union[int, None] = 2, hidden_dim_node_decoder: int = 128,
                 num_layers_node_decoder: Union[int, None] = 2, aggregation: Literal["sum", "mean"] = "sum",
                 do_concat_trick: bool = False, num_processor_checkpoint_segments: int = 0,
                 checkpoint_offloading: bool = False, recompute_activation: bool = False,
                 norm_type: Literal["LayerNorm", "TELayerNorm"] = "LayerNorm"):
        if do_concat_trick:
            raise NotImplementedError("Concat trick is not supported for HybridMeshGraphNet yet.")
        if recompute_activation:
            raise NotImplementedError("Recompute activation is not supported for HybridMeshGraphNet yet.")
        super().__init__(input_dim_nodes=input_dim_nodes, input_dim_edges=input_dim_edges, output_dim=output_dim,
                         processor_size=processor_size, mlp_activation_fn=mlp_activation_fn,
                         num_layers_node_processor=num_layers_node_processor,
                         num_layers_edge_processor=num_layers_edge_processor, hidden_dim_processor=hidden_dim_processor,
                         hidden_dim_node_encoder=hidden_dim_node_encoder, num_layers_node_encoder=num_layers_node_encoder,
                         hidden_dim_edge_encoder=hidden_dim_edge_encoder, num_layers_edge_encoder=num_layers_edge_encoder,
                         hidden_dim_node_decoder=hidden_dim_node_decoder, num_layers_node_decoder=num_layers_node_decoder,
                         aggregation=aggregation, do_concat_trick=do_concat_trick,
                         num_processor_checkpoint_segments=num_processor_checkpoint_segments,
                         checkpoint_offloading=checkpoint_offloading, recompute_activation=recompute_activation,
                         norm_type=norm_type)
        self.meta = _VariantMetaData()
        act = get_activation(mlp_activation_fn)
        self.mesh_edge_encoder = self.edge_encoder
        del self.edge_encoder
        self.world_edge_encoder = MeshGraphMLP(input_dim_edges, output_dim=hidden_dim_processor,
                                               hidden_dim=hidden_dim_edge_encoder, hidden_layers=num_layers_edge_encoder,
                                               activation_fn=act, norm_type=norm_type, recompute_activation=recompute_activation)
        self.processor = HybridMeshGraphNetProcessor(
            processor_size=processor_size, input_dim_node=hidden_dim_processor, input_dim_edge=hidden_dim_processor,
            num_layers_node=num_layers_node_processor, num_layers_edge=num_layers_edge_processor, aggregation=aggregation,
            norm_type=norm_type, activation_fn=act, do_concat_trick=do_concat_trick,
            num_processor_checkpoint_segments=num_processor_checkpoint_segments, checkpoint_offloading=checkpoint_offloading)

    def forward(self, node_features: Tensor, mesh_edge_features: Tensor, world_edge_features: Tensor, graph, **kwargs) -> Tensor:
        _check(node_features, self.input_dim_nodes, "N_nodes")
        _check(mesh_edge_features, self.input_dim_edges, "N_mesh_edges")
        _check(world_edge_features, self.input_dim_edges, "N_world_edges")
        x = self.processor(self.node_encoder(node_features), self.mesh_edge_encoder(mesh_edge_features),
                           self.world_edge_encoder(world_edge_features), graph)
        return self.node_decoder(x)
