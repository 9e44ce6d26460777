"""Graph construction back-end of GraphCast on the package's own ``Graph`` container.

Parity: ``physicsnemo/models/graphcast/utils/graph_backend.py`` (``PyGGraphBackend``:
``create_graph``, ``create_heterograph``, ``add_edge_features``, ``add_node_features``,
``khop_adj_all_k``).  The reference stores graphs as PyTorch-Geometric ``Data`` / ``HeteroData``;
here they are ``nn.module.gnn_layers.Graph`` objects (``edge_index`` plus source / destination
node counts, ``x``, ``edge_attr`` attributes), which every GNN layer of this package accepts, so
neither PyG nor ``torch_sparse`` is needed.

Edge features follow the GraphCast convention: both endpoints are rotated so that the receiver
sits at ``(1, 0, 0)``; the feature is the sender's displacement in that frame and its length,
optionally divided by the longest edge.  Node features are ``(cos lat, sin lon, cos lon)`` of the
coordinates in degrees passed to the trigonometric functions unchanged — kept that way because
trained weights depend on it.
"""
from __future__ import annotations

from typing import Tuple, Union

import numpy as np
import torch
from torch import Tensor

from ....nn.module.gnn_layers.graph_types import Graph as GraphData
from .graph_utils import azimuthal_angle, geospatial_rotation, polar_angle, xyz2latlon


class NativeGraphBackend:
    name: str = "pyg"          # the reference's only back-end name; graphs built here are drop-in for it

    @staticmethod
    def create_graph(src, dst, to_bidirected: bool, add_self_loop: bool, dtype: torch.dtype = torch.int64,
                     num_nodes: int | None = None) -> GraphData:
        src, dst = torch.as_tensor(np.asarray(src)).long(), torch.as_tensor(np.asarray(dst)).long()
        n = int(max(src.max(), dst.max())) + 1 if num_nodes is None else num_nodes
        if to_bidirected:                       # union with the reversed edges, duplicates removed, sorted by (src, dst)
            key = torch.unique(torch.cat([src * n + dst, dst * n + src]))
            src, dst = key // n, key % n
        if add_self_loop:
            keep = src != dst
            loops = torch.arange(n)
            src, dst = torch.cat([src[keep], loops]), torch.cat([dst[keep], loops])
        return GraphData(torch.stack([src, dst]), num_nodes=n)

    @staticmethod
    def create_heterograph(src, dst, labels, dtype: torch.dtype = torch.int64, num_src_nodes: int | None = None,
                           num_dst_nodes: int | None = None) -> GraphData:
        src, dst = torch.as_tensor(np.asarray(src)).long(), torch.as_tensor(np.asarray(dst)).long()
        ns = int(src.max()) + 1 if num_src_nodes is None else num_src_nodes
        nd = int(dst.max()) + 1 if num_dst_nodes is None else num_dst_nodes
        return GraphData(torch.stack([src, dst]), num_nodes=max(ns, nd), num_src_nodes=ns, num_dst_nodes=nd, labels=labels)

    @staticmethod
    def add_edge_features(graph: GraphData, pos: Union[Tensor, Tuple[Tensor, Tensor]], normalize: bool = True) -> GraphData:
        src_pos, dst_pos = pos if isinstance(pos, tuple) else (pos, pos)
        src, dst = graph.edge_index
        s, d = src_pos[src], dst_pos[dst]
        latlon = xyz2latlon(d, unit="rad")
        az, po = azimuthal_angle(latlon[:, 1]), polar_angle(latlon[:, 0])
        s = geospatial_rotation(geospatial_rotation(s, az, "z"), po, "y")
        d = geospatial_rotation(geospatial_rotation(d, az, "z"), po, "y")
        target = torch.tensor([1.0, 0.0, 0.0], dtype=d.dtype)
        if d.numel() and float((d - target).abs().max()) > 1e-4:
            raise ValueError("Invalid projection of edge nodes to local coordinate system")
        disp = s - d
        norm = torch.linalg.norm(disp, dim=-1, keepdim=True)
        if normalize:
            scale = norm.max()
            disp, norm = disp / scale, norm / scale
        graph.edge_attr = torch.cat((disp, norm), dim=-1)
        return graph

    @staticmethod
    def add_node_features(graph: GraphData, pos: Tensor) -> GraphData:
        latlon = xyz2latlon(pos)
        lat, lon = latlon[:, 0], latlon[:, 1]
        graph.x = torch.stack((torch.cos(lat), torch.sin(lon), torch.cos(lon)), dim=-1)
        return graph

    @staticmethod
    def khop_adj_all_k(graph: GraphData, kmax: int) -> Tensor:
        """Dense boolean ``[N, N]``: nodes within ``kmax`` hops of each other (walks of length 1..kmax)."""
        n = graph.num_nodes
        src, dst = graph.edge_index
        with torch.sparse.check_sparse_tensor_invariants(False):
            adj = torch.sparse_coo_tensor(torch.stack([src, dst]), torch.ones(src.numel()), (n, n)).coalesce()
        reach = adj.to_dense() > 0
        frontier = reach.clone()
        for _ in range(2, kmax + 1):
            frontier = (torch.sparse.mm(adj, frontier.float()) > 0)
            reach |= frontier
        return reach


PyGGraphBackend = NativeGraphBackend
