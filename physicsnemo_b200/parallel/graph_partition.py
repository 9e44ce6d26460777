"""Graph partition parallelism with the halo exchange fused into the message-passing gathers.

Reference behaviour: ``physicsnemo/nn/module/gnn_layers/distributed_graph.py:885-1197`` (``DistributedGraph``: node-wise
partition, halo source features fetched with ``indexed_all_to_all_v`` before every edge block, the reverse all-to-all +
``index_add_`` in backward, ``physicsnemo/distributed/utils.py:541-707``).

Here the graph is partitioned by destination node into contiguous blocks of a spatially sorted numbering: rank ``r``
owns nodes ``[start_r, start_{r+1})`` and every edge that ends in them.  Sources that belong to another rank are *halo*
nodes; locally they are numbered ``n_local + h``.  One step of message passing needs

* forward: the halo rows of the node features — read straight from the owner's memory inside the edge-gather kernel
  (``pnm_graph_gather_halo``; the owner first compacts its boundary rows into a mailbox, ``pnm_graph_halo_publish``);
* backward: the gradient rows of the halo nodes go back to their owners — every rank leaves them in its own mailbox
  and the owner of a boundary row adds up the copies of the peers that use it (``pnm_graph_halo_pull_add``).

On CPU (gloo) the same index structures drive ``all_gather`` based stand-ins, which is how the partition logic is
tested without GPUs.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from ..nn.module.gnn_layers.graph_types import Graph
from ..ops.graph import SegmentIndex


def split_sizes(n: int, parts: int) -> List[int]:
    """Block sizes of ``n`` items over ``parts`` ranks (ceil-sized chunks first, as ``compute_split_shapes``)."""
    from ..distributed.utils import compute_split_shapes

    return list(compute_split_shapes(n, parts))


class GraphPartitionPlan:
    """Index structures of ONE rank of a destination-owned partition (all NumPy, built once on the host)."""

    def __init__(self, rank: int, world: int, starts: np.ndarray, edge_src: np.ndarray, edge_dst: np.ndarray):
        self.rank, self.world = rank, world
        self.starts = starts                      # [world + 1] global node offsets
        lo, hi = int(starts[rank]), int(starts[rank + 1])
        self.n_local = hi - lo
        owner = lambda ids: np.searchsorted(starts[1:], ids, side="right")  # noqa: E731
        o_src, o_dst = owner(edge_src), owner(edge_dst)
        cross = o_src != o_dst
        # unique (consumer rank, source id) pairs over the whole graph, sorted by consumer then id
        n = int(starts[-1])
        key = np.unique(o_dst[cross].astype(np.int64) * n + edge_src[cross].astype(np.int64))
        pair_c, pair_id = key // n, key % n
        pair_o = owner(pair_id)
        # halo list of every consumer / send list of every owner
        halo_ids = [pair_id[pair_c == c] for c in range(world)]               # sorted by id (hence grouped by owner)
        send_ids = [np.unique(pair_id[pair_o == o]) for o in range(world)]
        self.n_send_all = [len(s) for s in send_ids]
        self.n_halo_all = [len(h) for h in halo_ids]
        my_halo = halo_ids[rank]
        self.n_halo = len(my_halo)
        self.halo_owner = owner(my_halo).astype(np.int32)
        self.halo_slot = np.zeros(self.n_halo, dtype=np.int32)
        for o in range(world):
            m = self.halo_owner == o
            if m.any():
                self.halo_slot[m] = np.searchsorted(send_ids[o], my_halo[m]).astype(np.int32)
        # local edges: destination owned here; sources renumbered into [0, n_local) U n_local + [0, n_halo)
        mine = o_dst == rank
        self.edge_ids = np.nonzero(mine)[0]                                    # positions in the global edge list
        s, d = edge_src[mine], edge_dst[mine]
        local_src = np.where(o_src[mine] == rank, s - lo, self.n_local + np.searchsorted(my_halo, s))
        self.edge_index = np.stack([local_src, d - lo]).astype(np.int64)
        # rows of mine that peers need, and for each of them the (peer, halo index at that peer) entries
        self.send_idx = (send_ids[rank] - lo).astype(np.int32)
        sel = pair_o == rank
        ent_c, ent_id = pair_c[sel], pair_id[sel]
        ent_h = np.zeros(len(ent_id), dtype=np.int64)
        for c in range(world):
            m = ent_c == c
            if m.any():
                ent_h[m] = np.searchsorted(halo_ids[c], ent_id[m])
        b = np.searchsorted(send_ids[rank], ent_id)
        order = np.argsort(b, kind="stable")
        self.ent_peer = ent_c[order].astype(np.int32)
        self.ent_slot = ent_h[order].astype(np.int32)
        counts = np.bincount(b, minlength=len(send_ids[rank]))
        self.bnd_off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        self.node_range = (lo, hi)


def plan_partition(edge_index: np.ndarray, num_nodes: int, world: int, rank: int) -> GraphPartitionPlan:
    """Partition plan of ``rank`` for a graph whose node numbering is already spatially sorted (block ownership)."""
    sizes = split_sizes(num_nodes, world)
    starts = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    return GraphPartitionPlan(rank, world, starts, np.asarray(edge_index[0]), np.asarray(edge_index[1]))


def spatial_order(coords: np.ndarray) -> np.ndarray:
    """Permutation that sorts the nodes into vertical strips (by the first coordinate): block ownership of the sorted
    numbering then cuts the domain into ``world`` strips with short boundaries."""
    return np.argsort(coords[:, 0], kind="stable")


class PartitionedGraph(Graph):
    """This rank's part of a partitioned graph, usable wherever the GNN layers take a ``Graph``.

    ``edge_index[0]`` (sources) indexes ``[0, n_local + n_halo)``; ``edge_index[1]`` the local nodes.  The layers call
    ``gather_src`` for the source features, everything else (destination gather, aggregation) is local.
    """

    def __init__(self, plan: GraphPartitionPlan, device, group: Optional[dist.ProcessGroup] = None, feature_dim: int = 128):
        ei = torch.from_numpy(plan.edge_index).to(device)
        super().__init__(ei, num_nodes=plan.n_local, num_src_nodes=plan.n_local + plan.n_halo, num_dst_nodes=plan.n_local)
        self.plan = plan
        self.group = group
        self.world, self.rank = plan.world, plan.rank
        self.n_local, self.n_halo = plan.n_local, plan.n_halo
        self.n_send = len(plan.send_idx)
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=torch.int32)  # noqa: E731
        self.src32 = ei[0].to(torch.int32).contiguous()
        self.halo_owner, self.halo_slot = i32(plan.halo_owner), i32(plan.halo_slot)
        self.send_idx = i32(plan.send_idx)
        self.bnd_off, self.ent_peer, self.ent_slot = i32(plan.bnd_off), i32(plan.ent_peer), i32(plan.ent_slot)
        self.src_segments = SegmentIndex(ei[0], plan.n_local + plan.n_halo)
        self.max_rows = max(max(plan.n_send_all), max(plan.n_halo_all), 1)
        self.feature_dim = feature_dim
        self._regions = None
        self._counter = None
        if self.world > 1 and torch.device(device).type == "cuda":
            from .peer import PeerRegions, peer_available

            if peer_available():
                self._regions = PeerRegions(group, region_floats=self.max_rows * feature_dim // 2 + 64, n_regions=4)
                self._counter = torch.zeros(4, dtype=torch.int32, device=device)

    def gather_src(self, nfeat: torch.Tensor) -> torch.Tensor:
        """``nfeat_global[src]`` for every local edge: local rows from ``nfeat``, halo rows from their owners."""
        if self.world == 1:
            from ..ops.graph import gather_rows

            return gather_rows(nfeat, self.src_segments)
        if self._regions is not None and nfeat.dtype == torch.bfloat16 and nfeat.shape[1] % 8 == 0:
            return _HaloGatherPeer.apply(nfeat, self)
        return _HaloGatherCollective.apply(nfeat, self)

    def step_done(self) -> None:
        if self._regions is not None:
            self._regions.step_done()


def _lib_gh():
    from ..ops import _lib

    lib = _lib.load(required=True)
    if not getattr(lib, "_gh_declared", False):
        c = ctypes
        vp, i, u, ll, d = c.c_void_p, c.c_int, c.c_uint, c.c_longlong, c.c_double
        lib.pnm_graph_halo_publish.argtypes = [vp, i, vp, vp, ll, i, vp, i, i, u, ll, vp, vp, vp]
        lib.pnm_graph_gather_halo.argtypes = [vp, i, vp, i, vp, vp, vp, vp, i, ll, i, i, vp, i, i, u, ll, d, vp, vp]
        lib.pnm_graph_halo_pull_add.argtypes = [vp, i, vp, vp, vp, vp, vp, ll, i, i, vp, i, i, u, ll, d, vp, vp]
        for n in ("pnm_graph_halo_publish", "pnm_graph_gather_halo", "pnm_graph_halo_pull_add"):
            getattr(lib, n).restype = i
        lib._gh_declared = True
    return lib


def _mailboxes(ptrs: Sequence[int], world: int):
    ptrs = list(ptrs) if len(ptrs) == world else [ptrs[0]] * world   # loopback: every "peer" is this rank's own mailbox
    ptrs = ptrs + [ptrs[0]] * (8 - len(ptrs))                         # the kernels take eight entries
    return (ctypes.c_void_p * 8)(*ptrs)


class _HaloGatherPeer(torch.autograd.Function):
    """Source gather with peer-memory halo reads (forward) and pull-model halo gradient sums (backward)."""

    @staticmethod
    def forward(ctx, nfeat, pg: PartitionedGraph):
        from ..ops import gemm as _g

        lib = _lib_gh()
        x = nfeat if (nfeat.stride(1) == 1 and nfeat.stride(0) % 8 == 0) else nfeat.contiguous()
        C = x.shape[1]
        reg = pg._regions
        view, ptrs = reg.region(pg.max_rows * C // 2, x.device)
        rt = reg.rt
        epoch = rt.next_epoch()
        bases, rank, world, ep, cap, budget, ebase = rt.peer_args(epoch)
        st = torch.cuda.current_stream().cuda_stream
        err = lib.pnm_graph_halo_publish(x.data_ptr(), x.stride(0), pg.send_idx.data_ptr(), view.data_ptr(), pg.n_send, C,
                                         bases, rank, world, ep, cap, ebase, pg._counter.data_ptr(), st)
        _g._check(err, "pnm_graph_halo_publish")
        E = pg.src32.numel()
        out = torch.empty(E, C, dtype=torch.bfloat16, device=x.device)
        err = lib.pnm_graph_gather_halo(x.data_ptr(), x.stride(0), pg.src32.data_ptr(), pg.n_local, pg.halo_owner.data_ptr(),
                                        pg.halo_slot.data_ptr(), _mailboxes(ptrs, pg.world), out.data_ptr(), out.stride(0), E, C, 1,
                                        bases, rank, world, ep, cap, budget, ebase, st)
        _g._check(err, "pnm_graph_gather_halo")
        _g.launch_count += 2
        ctx.pg = pg
        ctx.rows = x.shape[0]
        return out

    @staticmethod
    def backward(ctx, g):
        from ..ops import gemm as _g
        from ..ops.graph import _ok

        pg = ctx.pg
        lib = _lib_gh()
        g = _ok(g)
        C = g.shape[1]
        seg = pg.src_segments
        reg = pg._regions
        view, ptrs = reg.region(pg.max_rows * C // 2, g.device)
        dn = torch.empty(ctx.rows, C, dtype=torch.bfloat16, device=g.device)
        st = torch.cuda.current_stream().cuda_stream
        # sorted segment sums: local nodes into dn, halo nodes into this rank's mailbox (rows = halo index)
        code = lib.pnm_segment_sum(g.data_ptr(), g.stride(0), seg.perm.data_ptr(), seg.offsets.data_ptr(), dn.data_ptr(),
                                   dn.stride(0), pg.n_local, C, 0, 0, st)
        _g._check(code, "pnm_segment_sum")
        if pg.n_halo:
            code = lib.pnm_segment_sum(g.data_ptr(), g.stride(0), seg.perm.data_ptr(), seg.offsets.data_ptr() + 4 * pg.n_local,
                                       view.data_ptr(), C, pg.n_halo, C, 0, 0, st)
            _g._check(code, "pnm_segment_sum")
        peer = reg.publish()
        bases, rank, world, ep, cap, budget, ebase = peer
        err = lib.pnm_graph_halo_pull_add(dn.data_ptr(), dn.stride(0), pg.send_idx.data_ptr(), pg.bnd_off.data_ptr(),
                                          pg.ent_peer.data_ptr(), pg.ent_slot.data_ptr(), _mailboxes(ptrs, pg.world), pg.n_send, C,
                                          1, bases, rank, world, ep, cap, budget, ebase, st)
        _g._check(err, "pnm_graph_halo_pull_add")
        _g.launch_count += 4
        return dn, None


class _HaloGatherCollective(torch.autograd.Function):
    """The same exchange on ``torch.distributed`` collectives (CPU / gloo, or the selectable NCCL baseline)."""

    @staticmethod
    def forward(ctx, nfeat, pg: PartitionedGraph):
        C = nfeat.shape[1]
        mine = torch.zeros(pg.max_rows, C, dtype=nfeat.dtype, device=nfeat.device)
        if pg.n_send:
            mine[: pg.n_send] = nfeat[pg.send_idx.long()]
        boxes = [torch.empty_like(mine) for _ in range(pg.world)]
        dist.all_gather(boxes, mine, group=pg.group)
        allbox = torch.stack(boxes)                                            # [world, max_rows, C]
        halo = allbox[pg.halo_owner.long(), pg.halo_slot.long()] if pg.n_halo else nfeat.new_zeros(0, C)
        ext = torch.cat([nfeat, halo], dim=0)
        ctx.pg, ctx.rows = pg, nfeat.shape[0]
        return ext[pg.edge_index[0]]

    @staticmethod
    def backward(ctx, g):
        pg = ctx.pg
        C = g.shape[1]
        acc = torch.float32 if g.dtype in (torch.bfloat16, torch.float16) else g.dtype
        ext = torch.zeros(pg.n_local + pg.n_halo, C, dtype=acc, device=g.device)
        ext.index_add_(0, pg.edge_index[0], g.to(acc))
        mine = torch.zeros(pg.max_rows, C, dtype=acc, device=g.device)
        if pg.n_halo:
            mine[: pg.n_halo] = ext[pg.n_local:]
        boxes = [torch.empty_like(mine) for _ in range(pg.world)]
        dist.all_gather(boxes, mine, group=pg.group)
        allbox = torch.stack(boxes)
        dn = ext[: pg.n_local]
        if pg.n_send:
            contrib = allbox[pg.ent_peer.long(), pg.ent_slot.long()]          # one row per (boundary row, peer) entry
            counts = (pg.bnd_off[1:] - pg.bnd_off[:-1]).long()
            rows = torch.repeat_interleave(pg.send_idx.long(), counts)
            dn = dn.index_add(0, rows, contrib)
        return dn.to(g.dtype), None
