"""GraphCast: encode a lat-lon grid onto an icosahedral multimesh, process, decode back.

Parity: ``physicsnemo/models/graphcast/graph_cast_net.py`` (``GraphCastNet`` constructor arguments,
sub-module names ``encoder_embedder``, ``decoder_embedder``, ``encoder``, ``processor_encoder``,
``processor``, ``processor_decoder``, ``decoder``, ``finale``; ``encoder_forward`` /
``decoder_forward`` / ``custom_forward`` / ``forward``; checkpoint switches;
``get_lat_lon_partition_separators``).  Graphs are this package's ``Graph`` containers whose sorted
edge orders are cached, so aggregation runs on the segment-reduce kernels without atomics.
As in the reference's current back-end, the graph-partitioned mode (``partition_size > 1``) is
not available.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Literal, Optional, Tuple

import torch

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import get_activation
from ...nn.module.gnn_layers.embedder import GraphCastDecoderEmbedder, GraphCastEncoderEmbedder
from ...nn.module.gnn_layers.mesh_graph_decoder import MeshGraphDecoder
from ...nn.module.gnn_layers.mesh_graph_encoder import MeshGraphEncoder
from ...nn.module.gnn_layers.mesh_graph_mlp import MeshGraphMLP
from ...nn.module.gnn_layers.utils import set_checkpoint_fn
from .graph_cast_processor import GraphCastProcessor, GraphCastProcessorGraphTransformer
from .utils.graph import Graph

logger = logging.getLogger(__name__)


def get_lat_lon_partition_separators(partition_size: int) -> Tuple[list, list]:
    """Latitude / longitude box bounds splitting the globe into ``partition_size`` near-square chunks."""
    lat_chunks, lon_chunks, i = 1, partition_size, 0
    while lat_chunks < lon_chunks:
        i += 1
        if partition_size % i == 0:
            lat_chunks, lon_chunks = i, partition_size // i
    if lat_chunks * lon_chunks != partition_size:
        raise ValueError(f"Can't divide lat-lon grid into {lat_chunks} x {lon_chunks} chunks for partition_size={partition_size}.")
    dlat, dlon = 180.0 / lat_chunks, 360.0 / lon_chunks
    lo, hi = [], []
    for p_lat in range(lat_chunks):
        for p_lon in range(lon_chunks):
            lo.append([dlat * p_lat - 90.0, dlon * p_lon - 180.0])
            hi.append([dlat * (p_lat + 1) - 90.0, dlon * (p_lon + 1) - 180.0])
    hi[-1] = [None, None]
    return lo, hi


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


class GraphCastNet(Module):
    def __init__(self, mesh_level: Optional[int] = 6, multimesh: bool = True, input_res: tuple = (721, 1440),
                 input_dim_grid_nodes: int = 474, input_dim_mesh_nodes: int = 3, input_dim_edges: int = 4,
                 output_dim_grid_nodes: int = 227, processor_type: str = "MessagePassing", khop_neighbors: int = 32,
                 num_attention_heads: int = 4, processor_layers: int = 16, hidden_layers: int = 1, hidden_dim: int = 512,
                 aggregation: str = "sum", activation_fn: str = "silu", norm_type: str = "LayerNorm",
                 use_cugraphops_encoder: bool = False, use_cugraphops_processor: bool = False,
                 use_cugraphops_decoder: bool = False, do_concat_trick: bool = False, recompute_activation: bool = False,
                 partition_size: int = 1, partition_group_name: Optional[str] = None,
                 use_lat_lon_partitioning: bool = False, expect_partitioned_input: bool = False,
                 global_features_on_rank_0: bool = False, produce_aggregated_output: bool = True,
                 produce_aggregated_output_on_all_ranks: bool = True, graph_backend: Literal["dgl", "pyg"] = "pyg"):
        super().__init__(meta=MetaData())
        if use_cugraphops_encoder or use_cugraphops_processor or use_cugraphops_decoder:
            raise ImportError("cugraphops is deprecated and not supported for GraphCastNet.")
        if processor_type not in ("MessagePassing", "GraphTransformer"):
            raise ValueError(f"Invalid processor type {processor_type}")
        if graph_backend != "pyg":
            raise ValueError(f"Unsupported graph backend: {graph_backend}")
        if partition_size > 1:
            raise NotImplementedError("Distributed mode (partition_size > 1) is not supported by this graph back-end.")
        if processor_layers <= 2:
            raise ValueError("Expected at least 3 processor layers")
        self.processor_type = processor_type
        if processor_type == "MessagePassing":
            khop_neighbors = 0
        self.is_distributed = False
        self.expect_partitioned_input = expect_partitioned_input
        self.global_features_on_rank_0 = global_features_on_rank_0
        self.produce_aggregated_output = produce_aggregated_output
        self.produce_aggregated_output_on_all_ranks = produce_aggregated_output_on_all_ranks
        self.partition_group_name = partition_group_name
        self.graph_backend = graph_backend
        self.input_dim_grid_nodes, self.output_dim_grid_nodes, self.input_res = input_dim_grid_nodes, output_dim_grid_nodes, input_res

        self.latitudes = torch.linspace(-90, 90, steps=input_res[0])
        self.longitudes = torch.linspace(-180, 180, steps=input_res[1] + 1)[1:]
        self.lat_lon_grid = torch.stack(torch.meshgrid(self.latitudes, self.longitudes, indexing="ij"), dim=-1)
        self.graph = Graph(self.lat_lon_grid, mesh_level, multimesh, khop_neighbors, backend=graph_backend)
        self.mesh_graph, self.attn_mask = self.graph.create_mesh_graph(verbose=False)
        self.g2m_graph = self.graph.create_g2m_graph(verbose=False)
        self.m2g_graph = self.graph.create_m2g_graph(verbose=False)
        self.g2m_edata, self.m2g_edata, self.mesh_ndata = self.g2m_graph.edge_attr, self.m2g_graph.edge_attr, self.mesh_graph.x
        self.mesh_edata = (self.mesh_graph.edge_attr if processor_type == "MessagePassing"
                           else torch.zeros((1, input_dim_edges)))

        act = get_activation(activation_fn)
        self.model_checkpoint_fn = set_checkpoint_fn(False)
        self.encoder_checkpoint_fn = set_checkpoint_fn(False)
        self.decoder_checkpoint_fn = set_checkpoint_fn(False)
        mlp_kw = dict(hidden_dim=hidden_dim, hidden_layers=hidden_layers, activation_fn=act, norm_type=norm_type,
                      recompute_activation=recompute_activation)
        self.encoder_embedder = GraphCastEncoderEmbedder(input_dim_grid_nodes=input_dim_grid_nodes,
                                                         input_dim_mesh_nodes=input_dim_mesh_nodes,
                                                         input_dim_edges=input_dim_edges, output_dim=hidden_dim, **mlp_kw)
        self.decoder_embedder = GraphCastDecoderEmbedder(input_dim_edges=input_dim_edges, output_dim=hidden_dim, **mlp_kw)
        self.encoder = MeshGraphEncoder(aggregation=aggregation, input_dim_src_nodes=hidden_dim, input_dim_dst_nodes=hidden_dim,
                                        input_dim_edges=hidden_dim, output_dim_src_nodes=hidden_dim,
                                        output_dim_dst_nodes=hidden_dim, output_dim_edges=hidden_dim,
                                        do_concat_trick=do_concat_trick, **mlp_kw)
        if processor_type == "MessagePassing":
            def proc(n):
                return GraphCastProcessor(aggregation=aggregation, processor_layers=n, input_dim_nodes=hidden_dim,
                                          input_dim_edges=hidden_dim, do_concat_trick=do_concat_trick, **mlp_kw)

            self.processor_encoder, self.processor, self.processor_decoder = proc(1), proc(processor_layers - 2), proc(1)
        else:
            self.processor_encoder = torch.nn.Identity()
            self.processor = GraphCastProcessorGraphTransformer(attention_mask=self.attn_mask,
                                                                num_attention_heads=num_attention_heads,
                                                                processor_layers=processor_layers,
                                                                input_dim_nodes=hidden_dim, hidden_dim=hidden_dim)
            self.processor_decoder = torch.nn.Identity()
        self.decoder = MeshGraphDecoder(aggregation=aggregation, input_dim_src_nodes=hidden_dim, input_dim_dst_nodes=hidden_dim,
                                        input_dim_edges=hidden_dim, output_dim_dst_nodes=hidden_dim,
                                        output_dim_edges=hidden_dim, do_concat_trick=do_concat_trick, **mlp_kw)
        self.finale = MeshGraphMLP(input_dim=hidden_dim, output_dim=output_dim_grid_nodes, hidden_dim=hidden_dim,
                                   hidden_layers=hidden_layers, activation_fn=act, norm_type=None,
                                   recompute_activation=recompute_activation)

    # ---- activation checkpoint switches ----------------------------------------------------------------
    def set_checkpoint_model(self, checkpoint_flag: bool):
        self.model_checkpoint_fn = set_checkpoint_fn(checkpoint_flag)
        if checkpoint_flag:
            if hasattr(self.processor, "set_checkpoint_segments"):
                self.processor.set_checkpoint_segments(-1)
            self.encoder_checkpoint_fn = set_checkpoint_fn(False)
            self.decoder_checkpoint_fn = set_checkpoint_fn(False)

    def set_checkpoint_processor(self, checkpoint_segments: int):
        self.processor.set_checkpoint_segments(checkpoint_segments)

    def set_checkpoint_encoder(self, checkpoint_flag: bool):
        self.encoder_checkpoint_fn = set_checkpoint_fn(checkpoint_flag)

    def set_checkpoint_decoder(self, checkpoint_flag: bool):
        self.decoder_checkpoint_fn = set_checkpoint_fn(checkpoint_flag)

    # ---- stages ----------------------------------------------------------------------------------------
    def _check_features(self, t: torch.Tensor, width: int, what: str) -> None:
        if not torch.compiler.is_compiling() and (t.ndim != 2 or t.shape[1] != width):
            raise ValueError(f"Expected tensor of shape (N_grid, {what}) but got tensor of shape {tuple(t.shape)}")

    def encoder_forward(self, grid_nfeat):
        self._check_features(grid_nfeat, self.input_dim_grid_nodes, "C_in")
        dt = grid_nfeat.dtype
        grid_e, mesh_e, g2m_e, mesh_edge_e = self.encoder_embedder(grid_nfeat, self.mesh_ndata.to(dt), self.g2m_edata.to(dt),
                                                                   self.mesh_edata.to(dt))
        grid_enc, mesh_enc = self.encoder(g2m_e, grid_e, mesh_e, self.g2m_graph)
        if self.processor_type == "MessagePassing":
            mesh_efeat, mesh_nfeat = self.processor_encoder(mesh_edge_e, mesh_enc, self.mesh_graph)
        else:
            mesh_efeat, mesh_nfeat = None, self.processor_encoder(mesh_enc)
        return mesh_efeat, mesh_nfeat, grid_enc

    def decoder_forward(self, mesh_efeat_processed, mesh_nfeat_processed, grid_nfeat_encoded):
        if not torch.compiler.is_compiling():
            if mesh_nfeat_processed.ndim != 2:
                raise ValueError(f"Expected tensor of shape (N_mesh, C_hid) but got tensor of shape {tuple(mesh_nfeat_processed.shape)}")
            if grid_nfeat_encoded.ndim != 2:
                raise ValueError(f"Expected tensor of shape (N_grid, C_hid) but got tensor of shape {tuple(grid_nfeat_encoded.shape)}")
            if self.processor_type == "MessagePassing" and (mesh_efeat_processed is None or mesh_efeat_processed.ndim != 2):
                shape = None if mesh_efeat_processed is None else tuple(mesh_efeat_processed.shape)
                raise ValueError(f"Expected tensor of shape (N_mesh_edge, C_hid) but got tensor of shape {shape}")
        if self.processor_type == "MessagePassing":
            _, mesh_nfeat_processed = self.processor_decoder(mesh_efeat_processed, mesh_nfeat_processed, self.mesh_graph)
        else:
            mesh_nfeat_processed = self.processor_decoder(mesh_nfeat_processed)
        m2g_e = self.decoder_embedder(self.m2g_edata.to(grid_nfeat_encoded.dtype))
        return self.finale(self.decoder(m2g_e, grid_nfeat_encoded, mesh_nfeat_processed, self.m2g_graph))

    def custom_forward(self, grid_nfeat):
        self._check_features(grid_nfeat, self.input_dim_grid_nodes, "C_in")
        mesh_efeat, mesh_nfeat, grid_enc = self.encoder_checkpoint_fn(self.encoder_forward, grid_nfeat, use_reentrant=False,
                                                                      preserve_rng_state=False)
        if self.processor_type == "MessagePassing":
            mesh_efeat, mesh_nfeat = self.processor(mesh_efeat, mesh_nfeat, self.mesh_graph)
        else:
            mesh_efeat, mesh_nfeat = None, self.processor(mesh_nfeat)
        return self.decoder_checkpoint_fn(self.decoder_forward, mesh_efeat, mesh_nfeat, grid_enc, use_reentrant=False,
                                          preserve_rng_state=False)

    def forward(self, grid_nfeat):
        invar = self.prepare_input(grid_nfeat, self.expect_partitioned_input, self.global_features_on_rank_0)
        outvar = self.model_checkpoint_fn(self.custom_forward, invar, use_reentrant=False, preserve_rng_state=False)
        return self.prepare_output(outvar, self.produce_aggregated_output, self.produce_aggregated_output_on_all_ranks)

    def prepare_input(self, invar, expect_partitioned_input: bool, global_features_on_rank_0: bool):
        if global_features_on_rank_0 and expect_partitioned_input:
            raise ValueError("global_features_on_rank_0 and expect_partitioned_input cannot be set at the same time.")
        if not torch.compiler.is_compiling():
            want = (invar.shape[0], self.input_dim_grid_nodes, *self.input_res)
            if invar.ndim != 4 or tuple(invar.shape) != want:
                raise ValueError(f"Expected tensor of shape {want} but got tensor of shape {tuple(invar.shape)}")
        if invar.size(0) != 1:
            raise ValueError("GraphCast does not support batch size > 1. Expected tensor of shape (1, C_in, H, W) but got "
                             f"tensor of shape {tuple(invar.shape)}")
        return invar[0].reshape(self.input_dim_grid_nodes, -1).permute(1, 0)

    def prepare_output(self, outvar, produce_aggregated_output: bool, produce_aggregated_output_on_all_ranks: bool = True):
        self._check_features(outvar, self.output_dim_grid_nodes, "C_out")
        return outvar.permute(1, 0).reshape(self.output_dim_grid_nodes, *self.input_res).unsqueeze(0)

    def to(self, *args: Any, **kwargs: Any):
        self = super().to(*args, **kwargs)
        device, dtype, _, _ = torch._C._nn._parse_to(*args, **kwargs)
        for name in ("g2m_edata", "m2g_edata", "mesh_ndata", "mesh_edata"):
            setattr(self, name, getattr(self, name).to(*args, **kwargs))
        if device is not None:
            self.g2m_graph, self.mesh_graph, self.m2g_graph = (g.to(device) for g in (self.g2m_graph, self.mesh_graph, self.m2g_graph))
        return self
