"""Bi-stride multi-scale graphs (BSMS-GNN) over any graph dataset.

Parity: ``physicsnemo/datapipes/gnn/bsms.py`` (``BistrideMultiLayerGraph`` / ``BistrideMultiLayerGraphDataset``).  A
coarser level keeps every second breadth-first "stride" of the level below: in each connected component a search starts
at the node nearest to the component's centroid, nodes at even distance and nodes at odd distance form two sets, the
smaller (non-empty) one of which survives; survivors are linked when they were at most two hops apart.  The search runs
as frontier expansion on index tensors (all components at once), the two-hop closure is one sparse product.
"""
from __future__ import annotations

import pickle
from pathlib import Path
from typing import List, Optional, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset


def _components(n: int, src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """Component label (smallest node id of the component) of every node, by min-label propagation."""
    label = torch.arange(n)
    while True:
        new = label.clone()
        new.scatter_reduce_(0, dst, label[src], reduce="amin")
        new.scatter_reduce_(0, src, label[dst], reduce="amin")
        new = torch.minimum(new, new[new])                      # pointer jumping
        if torch.equal(new, label):
            return label
        label = new


def _bfs_parity(n: int, src: torch.Tensor, dst: torch.Tensor, seeds: torch.Tensor) -> torch.Tensor:
    """Breadth-first distance from the nearest seed (−1 where unreachable)."""
    dist = torch.full((n,), -1, dtype=torch.long)
    dist[seeds] = 0
    frontier = torch.zeros(n, dtype=torch.bool)
    frontier[seeds] = True
    level = 0
    while frontier.any():
        level += 1
        reach = torch.zeros(n, dtype=torch.bool)
        reach[dst[frontier[src]]] = True
        reach[src[frontier[dst]]] = True
        frontier = reach & (dist < 0)
        dist[frontier] = level
    return dist


def bistride_select(edge_index: torch.Tensor, pos: torch.Tensor, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """One coarsening step: ``(kept node ids (sorted), edge_index of the coarse graph in the new numbering)``."""
    import scipy.sparse as sp

    src, dst = edge_index[0].long(), edge_index[1].long()
    label = _components(n, src, dst)
    comp_ids, comp_of = torch.unique(label, return_inverse=True)
    C = comp_ids.numel()
    ones = torch.ones(n, dtype=pos.dtype)
    count = torch.zeros(C, dtype=pos.dtype).index_add_(0, comp_of, ones)
    centroid = torch.zeros(C, pos.shape[1], dtype=pos.dtype).index_add_(0, comp_of, pos) / count[:, None]
    d2 = (pos - centroid[comp_of]).square().sum(1)
    best = torch.full((C,), float("inf"), dtype=pos.dtype).scatter_reduce_(0, comp_of, d2, reduce="amin")
    cand = torch.nonzero(d2 <= best[comp_of]).reshape(-1)
    seeds = torch.full((C,), n, dtype=torch.long).scatter_reduce_(0, comp_of[cand], cand, reduce="amin")
    dist = _bfs_parity(n, src, dst, seeds)
    even = (dist >= 0) & (dist % 2 == 0)
    odd = (dist >= 0) & (dist % 2 == 1)
    n_even = torch.zeros(C, dtype=torch.long).index_add_(0, comp_of, even.long())
    n_odd = torch.zeros(C, dtype=torch.long).index_add_(0, comp_of, odd.long())
    keep_even = (n_even <= n_odd) | (n_odd == 0)
    kept_mask = torch.where(keep_even[comp_of], even, odd)
    kept = torch.nonzero(kept_mask).reshape(-1)
    a = sp.coo_matrix((np.ones(src.numel()), (src.numpy(), dst.numpy())), shape=(n, n)).tocsr()
    a = ((a + a.T) > 0).astype(np.float32) + sp.identity(n, dtype=np.float32, format="csr")
    two = (a @ a).tocoo()
    r, c = torch.as_tensor(two.row).long(), torch.as_tensor(two.col).long()
    new_id = torch.full((n,), -1, dtype=torch.long)
    new_id[kept] = torch.arange(kept.numel())
    ok = (r != c) & (new_id[r] >= 0) & (new_id[c] >= 0)
    return kept, torch.stack([new_id[r[ok]], new_id[c[ok]]])


class BistrideMultiLayerGraph:
    """``m_flat_es[l]``: edges of level ``l`` (level 0 = the input graph); ``m_ids[l]``: nodes of level ``l`` kept at
    level ``l + 1`` (ids in level ``l``'s numbering)."""

    def __init__(self, graph, num_layers: int):
        self.num_layers, self.num_nodes = num_layers, int(graph.num_nodes)
        edges = graph.edge_index.long().cpu()
        pos = graph.pos.detach().float().cpu()
        self.m_flat_es: List[torch.Tensor] = [edges]
        self.m_ids: List[torch.Tensor] = []
        n = self.num_nodes
        for _ in range(num_layers):
            kept, edges = bistride_select(edges, pos, n)
            pos, n = pos[kept], kept.numel()
            self.m_flat_es.append(edges)
            self.m_ids.append(kept)

    def get_multi_layer_graphs(self):
        return self.m_flat_es, self.m_flat_es, self.m_ids


class BistrideMultiLayerGraphDataset(Dataset):
    """Wraps a graph dataset: ``{"graph", "ms_edges", "ms_ids"}`` per sample; the hierarchy of a sample is cached on disk
    (it depends only on the mesh)."""

    def __init__(self, dataset: Dataset, num_layers: int = 1, cache_dir: Optional[str | Path] = None, **kwargs):
        self.dataset, self.num_layers = dataset, num_layers
        self.cache_dir = None
        if cache_dir is not None:
            self.cache_dir = Path(cache_dir) / str(getattr(dataset, "split", "all"))
            self.cache_dir.mkdir(parents=True, exist_ok=True)

    def __len__(self) -> int:
        return len(self.dataset)

    def __getattr__(self, name):
        if name in ("dataset", "num_layers", "cache_dir"):
            raise AttributeError(name)
        return getattr(self.dataset, name)

    def _cache_file(self, idx: int) -> Path:
        return self.cache_dir / f"{idx:03}.pkl"

    def __getitem__(self, idx: int):
        graph = self.dataset[idx]
        graph = graph[0] if isinstance(graph, tuple) else graph
        levels = None
        if self.cache_dir is not None and self._cache_file(idx).exists():
            with open(self._cache_file(idx), "rb") as f:
                levels = pickle.load(f)
        if levels is None:
            ms = BistrideMultiLayerGraph(graph, self.num_layers)
            levels = ([e.numpy() for e in ms.m_flat_es], [i.numpy() for i in ms.m_ids])
            if self.cache_dir is not None:
                with open(self._cache_file(idx), "wb") as f:
                    pickle.dump(levels, f)
        edges, ids = levels
        return {"graph": graph, "ms_edges": [torch.as_tensor(e, dtype=torch.long) for e in edges],
                "ms_ids": [torch.as_tensor(i, dtype=torch.long) for i in ids]}
