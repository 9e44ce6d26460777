"""The three graphs of GraphCast: multi-scale mesh, grid → mesh and mesh → grid.

Parity: ``physicsnemo/models/graphcast/utils/graph.py`` (``Graph``: ``create_mesh_graph``,
``create_g2m_graph``, ``create_m2g_graph``).  Grid → mesh edges join every grid point to those of
its 4 nearest mesh vertices that lie within 0.6 × the longest edge of the finest mesh; mesh → grid
edges join the three vertices of the face whose centroid is nearest to every grid point.  Nearest
neighbours come from this package's ``knn`` functional (a brute-force tiled kernel on a GPU, a
k-d tree on the CPU) and the edge lists are assembled with array operations.
"""
from __future__ import annotations

import logging

import numpy as np
import torch
from torch import Tensor

from .graph_backend import NativeGraphBackend
from .graph_utils import get_face_centroids, latlon2xyz, max_edge_length, xyz2latlon
from .icosahedral_mesh import faces_to_edges, get_hierarchy_of_triangular_meshes_for_sphere, merge_meshes

logger = logging.getLogger(__name__)


def _nearest(points: Tensor, queries: Tensor, k: int):
    from ....nn.functional.neighbors import knn

    idx, dist = knn(points.float(), queries.float(), k)
    return idx.long(), dist


class Graph:
    def __init__(self, lat_lon_grid: Tensor, mesh_level: int = 6, multimesh: bool = True, khop_neighbors: int = 0,
                 dtype=torch.float, backend: str = "pyg") -> None:
        if backend != "pyg":
            raise ValueError(f"Unsupported backend: {backend}")
        self.khop_neighbors = khop_neighbors
        self.dtype = dtype
        self.backend = NativeGraphBackend
        self.lat_lon_grid_flat = lat_lon_grid.permute(2, 0, 1).reshape(2, -1).permute(1, 0)
        meshes = get_hierarchy_of_triangular_meshes_for_sphere(splits=mesh_level)
        finest = meshes[-1]
        self.finest_mesh_src, self.finest_mesh_dst = faces_to_edges(finest.faces)
        self.finest_mesh_vertices = np.array(finest.vertices)
        mesh = merge_meshes(meshes) if multimesh else finest
        self.mesh_src, self.mesh_dst = faces_to_edges(mesh.faces)
        self.mesh_vertices = np.array(mesh.vertices)
        self.mesh_faces = mesh.faces

    def create_mesh_graph(self, verbose: bool = True):
        n = self.mesh_vertices.shape[0]
        g = self.backend.create_graph(self.mesh_src, self.mesh_dst, to_bidirected=True, add_self_loop=False, num_nodes=n)
        pos = torch.tensor(self.mesh_vertices, dtype=torch.float32)
        g = self.backend.add_node_features(self.backend.add_edge_features(g, pos), pos)
        g.lat_lon = xyz2latlon(pos)
        g.x, g.edge_attr = g.x.to(self.dtype), g.edge_attr.to(self.dtype)
        mask = ~self.backend.khop_adj_all_k(g, self.khop_neighbors) if self.khop_neighbors > 0 else None
        if verbose:
            print("mesh graph:", g.num_nodes, "nodes,", g.num_edges, "edges")
        return g, mask

    def _bipartite(self, src, dst, labels, src_pos: Tensor, dst_pos: Tensor, src_ll: Tensor, dst_ll: Tensor):
        g = self.backend.create_heterograph(src, dst, labels, num_src_nodes=src_pos.shape[0], num_dst_nodes=dst_pos.shape[0])
        g = self.backend.add_edge_features(g, (src_pos, dst_pos))
        g.src_pos, g.dst_pos = src_pos.to(self.dtype), dst_pos.to(self.dtype)
        g.src_lat_lon, g.dst_lat_lon = src_ll, dst_ll
        g.edge_attr = g.edge_attr.to(self.dtype)
        return g

    def create_g2m_graph(self, verbose: bool = True):
        limit = 0.6 * max_edge_length(self.finest_mesh_vertices, self.finest_mesh_src, self.finest_mesh_dst)
        grid = latlon2xyz(self.lat_lon_grid_flat).to(torch.float32)
        mesh = torch.tensor(self.mesh_vertices, dtype=torch.float32)
        idx, dist = _nearest(mesh, grid, 4)
        keep = dist <= limit
        src = torch.arange(grid.shape[0])[:, None].expand_as(idx)[keep]
        g = self._bipartite(src, idx[keep], ("grid", "g2m", "mesh"), grid, mesh, self.lat_lon_grid_flat, xyz2latlon(mesh))
        if verbose:
            print("g2m graph:", g.num_edges, "edges")
        return g

    def create_m2g_graph(self, verbose: bool = True):
        grid = latlon2xyz(self.lat_lon_grid_flat).to(torch.float32)
        mesh = torch.tensor(self.mesh_vertices, dtype=torch.float32)
        centroids = torch.tensor(get_face_centroids(self.mesh_vertices, self.mesh_faces), dtype=torch.float32)
        face, _ = _nearest(centroids, grid, 1)
        src = torch.as_tensor(np.asarray(self.mesh_faces)).long()[face[:, 0]].reshape(-1)     # 3 vertices per grid point
        dst = torch.arange(grid.shape[0]).repeat_interleave(3)
        g = self._bipartite(src, dst, ("mesh", "m2g", "grid"), mesh, grid, xyz2latlon(mesh), self.lat_lon_grid_flat)
        if verbose:
            print("m2g graph:", g.num_edges, "edges")
        return g
