"""Graph partitioning over ranks and the collectives that move node / edge features between layouts.

Parity: ``physicsnemo/nn/module/gnn_layers/distributed_graph.py`` (``GraphPartition``,
``partition_graph_with_id_mapping``, ``partition_graph_with_matrix_decomposition``,
``partition_graph_nodewise``, ``partition_graph_by_coordinate_bbox``, ``DistributedGraph``).

A graph is given in CSC form (``global_offsets [N_dst + 1]``, ``global_indices [E]`` = source of every
edge, edges grouped by destination).  Every rank owns a set of destination nodes with all their incoming
edges and a set of source nodes; the local graph of a rank refers to the distinct sources of its edges,
ordered by owning rank, so the features it needs from rank ``r`` form one contiguous block filled by a
single indexed all-to-all (``scatter_indices[r]`` = rows rank ``partition_rank`` sends to ``r``,
``sizes[from][to]`` = row counts).  The partitioners are array computations: edge lists of a set of
destinations are expanded with ``repeat_interleave`` and there is no per-node Python loop.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from ....distributed import DistributedManager, all_gather_v, gather_v, indexed_all_to_all_v, scatter_v

logger = logging.getLogger(__name__)


@dataclass
class GraphPartition:
    partition_size: int
    partition_rank: int
    device: torch.device
    matrix_decomp: bool = False
    local_offsets: Optional[torch.Tensor] = None
    local_indices: Optional[torch.Tensor] = None
    num_local_src_nodes: int = -1
    num_local_dst_nodes: int = -1
    num_local_indices: int = -1
    map_partitioned_src_ids_to_global: Optional[torch.Tensor] = None
    map_concatenated_local_src_ids_to_global: Optional[torch.Tensor] = None
    map_partitioned_dst_ids_to_global: Optional[torch.Tensor] = None
    map_concatenated_local_dst_ids_to_global: Optional[torch.Tensor] = None
    map_partitioned_edge_ids_to_global: Optional[torch.Tensor] = None
    map_concatenated_local_edge_ids_to_global: Optional[torch.Tensor] = None
    map_global_src_ids_to_concatenated_local: Optional[torch.Tensor] = None
    map_global_dst_ids_to_concatenated_local: Optional[torch.Tensor] = None
    map_global_edge_ids_to_concatenated_local: Optional[torch.Tensor] = None
    sizes: Optional[List[List[int]]] = None
    scatter_indices: Optional[List[torch.Tensor]] = None
    num_src_nodes_in_each_partition: Optional[List[int]] = None
    num_dst_nodes_in_each_partition: Optional[List[int]] = None
    num_indices_in_each_partition: Optional[List[int]] = None

    def __post_init__(self):
        p = self.partition_size
        if p <= 0:
            raise ValueError(f"Expected partition_size > 0, got {p}")
        if not 0 <= self.partition_rank < p:
            raise ValueError(f"Expected 0 <= partition_rank < {p}, got {self.partition_rank}")
        if self.sizes is None:
            self.sizes = [[None] * p for _ in range(p)]
        for name in ("scatter_indices", "num_src_nodes_in_each_partition", "num_dst_nodes_in_each_partition",
                     "num_indices_in_each_partition"):
            if getattr(self, name) is None:
                setattr(self, name, [None] * p)

    def to(self, *args, **kwargs):
        for name, value in list(vars(self).items()):
            if isinstance(value, torch.Tensor):
                setattr(self, name, value.to(*args, **kwargs))
        self.scatter_indices = [i.to(*args, **kwargs) if isinstance(i, torch.Tensor) else i for i in self.scatter_indices]
        return self

    def check(self) -> None:
        for r in range(self.partition_size):
            if self.sizes[self.partition_rank][r] != self.scatter_indices[r].numel():
                raise AssertionError("error in graph partition: list containing sizes of exchanged indices does not match "
                                     "the tensor of indices to be exchanged")


def _inverse_of(perm: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), dtype=perm.dtype, device=perm.device)
    return inv


def _edges_of(offsets: torch.Tensor, nodes: torch.Tensor):
    """Edge ids (grouped by node, in ``nodes`` order) and the local CSC offsets of a set of destination nodes."""
    start, deg = offsets[nodes], offsets[nodes + 1] - offsets[nodes]
    local_offsets = torch.cat([deg.new_zeros(1), deg.cumsum(0)])
    within = torch.arange(int(local_offsets[-1]), dtype=offsets.dtype, device=offsets.device) - local_offsets[:-1].repeat_interleave(deg)
    return start.repeat_interleave(deg) + within, local_offsets


def partition_graph_with_id_mapping(global_offsets: torch.Tensor, global_indices: torch.Tensor,
                                    mapping_src_ids_to_ranks: torch.Tensor, mapping_dst_ids_to_ranks: torch.Tensor,
                                    partition_size: int, partition_rank: int, device: torch.device) -> GraphPartition:
    gp = GraphPartition(partition_size=partition_size, partition_rank=partition_rank, device=device)
    dtype = global_indices.dtype
    src_rank, dst_rank = mapping_src_ids_to_ranks.long(), mapping_dst_ids_to_ranks.long()
    # concatenated-local numbering = nodes sorted by owning rank (stable: ascending global id within a rank)
    src_order = torch.argsort(src_rank, stable=True).to(dtype)
    dst_order = torch.argsort(dst_rank, stable=True).to(dtype)
    gp.map_concatenated_local_src_ids_to_global, gp.map_global_src_ids_to_concatenated_local = src_order, _inverse_of(src_order)
    gp.map_concatenated_local_dst_ids_to_global, gp.map_global_dst_ids_to_concatenated_local = dst_order, _inverse_of(dst_order)
    src_counts = torch.bincount(src_rank, minlength=partition_size)
    dst_counts = torch.bincount(dst_rank, minlength=partition_size)
    for name, counts in (("source", src_counts), ("destination", dst_counts)):
        empty = (counts == 0).nonzero()
        if empty.numel():
            raise RuntimeError(f"Aborting partitioning, rank {int(empty[0])} has 0 {name} nodes to work on.")
    gp.num_src_nodes_in_each_partition = src_counts.tolist()
    gp.num_dst_nodes_in_each_partition = dst_counts.tolist()
    src_starts = torch.cat([src_counts.new_zeros(1), src_counts.cumsum(0)])
    dst_starts = torch.cat([dst_counts.new_zeros(1), dst_counts.cumsum(0)])
    # position of every source node inside its owner's partition
    src_local = gp.map_global_src_ids_to_concatenated_local.long() - src_starts[src_rank]
    edge_blocks = []
    for rank in range(partition_size):
        dst_nodes = dst_order[dst_starts[rank]:dst_starts[rank + 1]].long()
        edge_ids, local_offsets = _edges_of(global_offsets.long(), dst_nodes)
        edge_blocks.append(edge_ids)
        src_of_edges = global_indices[edge_ids].long()
        uniq, _ = torch.unique(src_of_edges, sorted=True, return_inverse=True)
        owner = src_rank[uniq]
        by_owner = torch.argsort(owner, stable=True)                       # local-graph numbering: grouped by owner
        local_id = torch.empty_like(uniq)
        local_id[by_owner] = torch.arange(uniq.numel(), device=uniq.device)
        per_owner = torch.bincount(owner, minlength=partition_size)
        for owner_rank in range(partition_size):
            gp.sizes[owner_rank][rank] = int(per_owner[owner_rank])
        mine = owner == partition_rank
        gp.scatter_indices[rank] = src_local[uniq[mine]].to(torch.int64)    # rows this rank sends to `rank`
        gp.num_indices_in_each_partition[rank] = int(edge_ids.numel())
        if rank == partition_rank:
            lookup = torch.zeros(src_rank.numel(), dtype=torch.long, device=uniq.device)
            lookup[uniq] = local_id
            gp.local_offsets = local_offsets.to(dtype)
            gp.local_indices = lookup[src_of_edges].to(dtype)
            gp.num_local_indices = int(edge_ids.numel())
            gp.num_local_dst_nodes = int(dst_counts[rank])
            gp.num_local_src_nodes = int(uniq.numel())
            gp.map_partitioned_src_ids_to_global = src_order[src_starts[rank]:src_starts[rank + 1]]
            gp.map_partitioned_dst_ids_to_global = dst_nodes.to(dtype)
            gp.map_partitioned_edge_ids_to_global = edge_ids.to(dtype)
    edge_order = torch.cat(edge_blocks).to(dtype)
    gp.map_concatenated_local_edge_ids_to_global, gp.map_global_edge_ids_to_concatenated_local = edge_order, _inverse_of(edge_order)
    gp.check()
    return gp.to(device=device)


def partition_graph_with_matrix_decomposition(global_offsets: torch.Tensor, global_indices: torch.Tensor, num_nodes: int,
                                              partition_book: torch.Tensor, partition_size: int, partition_rank: int,
                                              device: torch.device) -> GraphPartition:
    """Contiguous row blocks of a square adjacency matrix: ranks own ``partition_book[r] .. partition_book[r+1]``."""
    gp = GraphPartition(partition_size=partition_size, partition_rank=partition_rank, device=device, matrix_decomp=True)
    dtype = global_indices.dtype
    book = partition_book.long()
    lo, hi = int(book[partition_rank]), int(book[partition_rank + 1])
    if hi > num_nodes:
        raise ValueError("Invalid node offset and number of local nodes")
    offsets = global_offsets.long()
    e0 = int(offsets[lo])
    gp.local_offsets = (offsets[lo:hi + 1] - e0).to(dtype)
    gp.num_local_dst_nodes = hi - lo
    for to in range(partition_size):
        block = global_indices[int(offsets[book[to]]):int(offsets[book[to + 1]])].long()
        uniq, inverse = torch.unique(block, sorted=True, return_inverse=True)
        owner = torch.bucketize(uniq, book, right=True) - 1
        gp.scatter_indices[to] = (uniq[owner == partition_rank] - lo).to(torch.int64)
        gp.num_indices_in_each_partition[to] = int(block.numel())
        gp.num_dst_nodes_in_each_partition[to] = int(book[to + 1] - book[to])
        gp.num_src_nodes_in_each_partition[to] = int(uniq.numel())
        per_owner = torch.bincount(owner, minlength=partition_size)
        for frm in range(partition_size):
            gp.sizes[frm][to] = int(per_owner[frm])
        if to == partition_rank:
            gp.local_indices = inverse.to(dtype)
            gp.num_local_indices = int(inverse.numel())
            gp.num_local_src_nodes = int(uniq.numel())
            gp.map_partitioned_src_ids_to_global = uniq.to(dtype)
    gp.map_partitioned_dst_ids_to_global = torch.arange(lo, hi, dtype=dtype)
    gp.map_partitioned_edge_ids_to_global = torch.arange(e0, e0 + gp.num_local_indices, dtype=dtype)
    ident_nodes = torch.arange(num_nodes, dtype=dtype)
    ident_edges = torch.arange(global_indices.numel(), dtype=dtype)
    for name in ("map_concatenated_local_src_ids_to_global", "map_concatenated_local_dst_ids_to_global",
                 "map_global_src_ids_to_concatenated_local", "map_global_dst_ids_to_concatenated_local"):
        setattr(gp, name, ident_nodes)
    gp.map_concatenated_local_edge_ids_to_global = gp.map_global_edge_ids_to_concatenated_local = ident_edges
    gp.check()
    return gp.to(device=device)


def partition_graph_nodewise(global_offsets: torch.Tensor, global_indices: torch.Tensor, partition_size: int,
                             partition_rank: int, device: torch.device, matrix_decomp: bool = False) -> GraphPartition:
    """Equal consecutive chunks of node ids per rank."""
    n_src = int(global_indices.max()) + 1
    n_dst = global_offsets.size(0) - 1
    dst_chunk = (n_dst + partition_size - 1) // partition_size
    if matrix_decomp:
        if n_src != n_dst:
            raise ValueError("Must be square adj. matrix (num_src=num_dst) for matrix decomposition")
        book = torch.cat([torch.arange(0, n_dst, dst_chunk, dtype=global_indices.dtype),
                          torch.tensor([n_dst], dtype=global_indices.dtype)])
        return partition_graph_with_matrix_decomposition(global_offsets, global_indices, n_dst, book, partition_size,
                                                         partition_rank, device)
    src_chunk = (n_src + partition_size - 1) // partition_size
    kw = dict(dtype=global_offsets.dtype, device=global_offsets.device)
    return partition_graph_with_id_mapping(global_offsets, global_indices, torch.arange(n_src, **kw) // src_chunk,
                                           torch.arange(n_dst, **kw) // dst_chunk, partition_size, partition_rank, device)


def partition_graph_by_coordinate_bbox(global_offsets: torch.Tensor, global_indices: torch.Tensor,
                                       src_coordinates: torch.Tensor, dst_coordinates: torch.Tensor,
                                       coordinate_separators_min: List[List[Optional[float]]],
                                       coordinate_separators_max: List[List[Optional[float]]], partition_size: int,
                                       partition_rank: int, device: torch.device) -> GraphPartition:
    """Ranks own the nodes inside their axis-aligned box ``[min, max)`` (``None`` = unbounded on that side)."""
    dim = src_coordinates.size(-1)
    if dst_coordinates.size(-1) != dim:
        raise ValueError("source and destination coordinates must have the same dimension")
    for name, seps in (("coordinate_separators_min", coordinate_separators_min), ("coordinate_separators_max", coordinate_separators_max)):
        if len(seps) != partition_size:
            raise ValueError(f"Expected len({name}) == partition_size, but got {len(seps)} and {partition_size} respectively")
        for r, s in enumerate(seps):
            if len(s) != dim:
                raise ValueError(f"Expected len({name}[{r}]) == dim, but got {len(s)} and {dim} respectively")

    def assign(coords: torch.Tensor, n: int) -> torch.Tensor:
        mapping = torch.zeros(n, dtype=global_offsets.dtype, device=global_offsets.device)
        for p in range(partition_size):
            mask = torch.ones(n, dtype=torch.bool, device=coords.device)
            for d in range(dim):
                lo, hi = coordinate_separators_min[p][d], coordinate_separators_max[p][d]
                if lo is not None:
                    mask &= coords[:, d] >= lo
                if hi is not None:
                    mask &= coords[:, d] < hi
            mapping[mask.to(mapping.device)] = p
        return mapping

    n_src = int(global_indices.max()) + 1
    n_dst = global_offsets.size(0) - 1
    return partition_graph_with_id_mapping(global_offsets, global_indices, assign(src_coordinates, n_src),
                                           assign(dst_coordinates, n_dst), partition_size, partition_rank, device)


class DistributedGraph:
    """Feature movement between the global, the partitioned and the local-graph layouts of a ``GraphPartition``."""

    def __init__(self, global_offsets: torch.Tensor, global_indices: torch.Tensor, partition_size: int,
                 graph_partition_group_name: str = None, graph_partition: Optional[GraphPartition] = None):
        dm = DistributedManager()
        self.device = dm.device
        self.partition_rank = dm.group_rank(name=graph_partition_group_name)
        self.partition_size = dm.group_size(name=graph_partition_group_name)
        if self.partition_size != partition_size:
            raise AssertionError(f"Passed partition_size does not correspond to size of process_group, got {partition_size} "
                                 f"and {self.partition_size} respectively.")
        self.process_group = dm.group(name=graph_partition_group_name)
        if graph_partition is None:
            graph_partition = partition_graph_nodewise(global_offsets, global_indices, self.partition_size,
                                                       self.partition_rank, self.device)
        else:
            if graph_partition.partition_size != self.partition_size:
                raise AssertionError("Passed graph_partition.partition_size does not correspond to size of process_group, got "
                                     f"{graph_partition.partition_size} and {self.partition_size} respectively.")
            if torch.device(graph_partition.device) != torch.device(self.device):
                raise AssertionError("Passed graph_partition.device does not correspond to device of this rank, got "
                                     f"{graph_partition.device} and {self.device} respectively.")
        self.graph_partition = gp = graph_partition
        logger.info("GraphPartition(rank=%d, local src %d, local dst %d, send %s, recv %s)", gp.partition_rank,
                    gp.num_local_src_nodes, gp.num_local_dst_nodes, gp.sizes[gp.partition_rank],
                    [row[gp.partition_rank] for row in gp.sizes])
        if dist.is_initialized():
            dist.barrier(self.process_group)

    # ---- global -> partition ----------------------------------------------------------------------------------
    def _to_partition(self, feats, concat_map, part_map, counts, scatter_features: bool, src_rank: int):
        if scatter_features:
            return scatter_v(feats.to(self.device)[concat_map], counts, dim=0, src=src_rank, group=self.process_group)
        return feats.to(device=self.device)[part_map]

    def get_src_node_features_in_partition(self, global_node_features, scatter_features: bool = False, src_rank: int = 0):
        gp = self.graph_partition
        if gp.matrix_decomp:
            return self.get_dst_node_features_in_partition(global_node_features, scatter_features, src_rank)
        return self._to_partition(global_node_features, gp.map_concatenated_local_src_ids_to_global,
                                  gp.map_partitioned_src_ids_to_global, gp.num_src_nodes_in_each_partition, scatter_features, src_rank)

    def get_dst_node_features_in_partition(self, global_node_features, scatter_features: bool = False, src_rank: int = 0):
        gp = self.graph_partition
        return self._to_partition(global_node_features, gp.map_concatenated_local_dst_ids_to_global,
                                  gp.map_partitioned_dst_ids_to_global, gp.num_dst_nodes_in_each_partition, scatter_features, src_rank)

    def get_edge_features_in_partition(self, global_edge_features, scatter_features: bool = False, src_rank: int = 0):
        gp = self.graph_partition
        return self._to_partition(global_edge_features, gp.map_concatenated_local_edge_ids_to_global,
                                  gp.map_partitioned_edge_ids_to_global, gp.num_indices_in_each_partition, scatter_features, src_rank)

    # ---- partition -> local graph ---------------------------------------------------------------------------------
    def get_src_node_features_in_local_graph(self, partitioned_src_node_features: torch.Tensor) -> torch.Tensor:
        """Halo gather: every rank receives the rows of the distinct sources of its edges (differentiable)."""
        gp = self.graph_partition
        return indexed_all_to_all_v(partitioned_src_node_features, indices=gp.scatter_indices, sizes=gp.sizes, use_fp32=True,
                                    dim=0, group=self.process_group)

    def get_dst_node_features_in_local_graph(self, partitioned_dst_node_features: torch.Tensor) -> torch.Tensor:
        return partitioned_dst_node_features

    def get_edge_features_in_local_graph(self, partitioned_edge_features: torch.Tensor) -> torch.Tensor:
        return partitioned_edge_features

    # ---- partition -> global --------------------------------------------------------------------------------------
    def _to_global(self, feats, counts, inverse_map, get_on_all_ranks: bool, dst_rank: int):
        if feats.device != torch.device(self.device) and str(feats.device) != str(self.device):
            raise AssertionError(f"Passed features are on {feats.device}, this rank works on {self.device}.")
        if not get_on_all_ranks:
            out = gather_v(feats, counts, dim=0, dst=dst_rank, group=self.process_group)
            return out[inverse_map] if self.graph_partition.partition_rank == dst_rank else out
        return all_gather_v(feats, counts, dim=0, use_fp32=True, group=self.process_group)[inverse_map]

    def get_global_src_node_features(self, partitioned_node_features, get_on_all_ranks: bool = True, dst_rank: int = 0):
        gp = self.graph_partition
        if gp.matrix_decomp:
            return self.get_global_dst_node_features(partitioned_node_features, get_on_all_ranks, dst_rank)
        return self._to_global(partitioned_node_features, gp.num_src_nodes_in_each_partition,
                               gp.map_global_src_ids_to_concatenated_local, get_on_all_ranks, dst_rank)

    def get_global_dst_node_features(self, partitioned_node_features, get_on_all_ranks: bool = True, dst_rank: int = 0):
        gp = self.graph_partition
        return self._to_global(partitioned_node_features, gp.num_dst_nodes_in_each_partition,
                               gp.map_global_dst_ids_to_concatenated_local, get_on_all_ranks, dst_rank)

    def get_global_edge_features(self, partitioned_edge_features, get_on_all_ranks: bool = True, dst_rank: int = 0):
        gp = self.graph_partition
        return self._to_global(partitioned_edge_features, gp.num_indices_in_each_partition,
                               gp.map_global_edge_ids_to_concatenated_local, get_on_all_ranks, dst_rank)
