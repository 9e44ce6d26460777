"""Cluster tree over a point set and the near / far interaction lists of a treecode.

Parity: ``physicsnemo/mesh/spatial/cluster_tree.py`` (``ClusterTree.from_points`` ``:649``,
``compute_source_aggregates`` ``:784``, ``find_dual_interaction_pairs`` ``:905``,
``DualInteractionPlan`` ``:67``).  The design here differs:

* the tree is a balanced binary tree made by median splits along the longest box axis, built level by
  level with two stable sorts per level (no Morton codes, no per-node Python loop);
* the traversal walks a (target node, source node) frontier level by level and emits two flat lists:
  ``near`` pairs of (target point, source point), evaluated exactly, and ``far`` pairs of
  (target point, source node), evaluated against the node's aggregate.  The target side is never
  approximated: a far node pair is expanded to the individual targets of the target node, which is
  the behaviour the reference reaches with ``expand_far_targets=True``;
* node sums (areas, centroids, averaged features, strengths) come from fp64 prefix sums over the
  tree order, because every node covers one contiguous range of it.

All steps are batched tensor operations, so the same code runs on the host or on the device that
holds the points.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch


def ragged_arange(starts: torch.Tensor, counts: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Concatenation of ``arange(s, s + c)`` over all rows, plus the row index of every element."""
    counts = counts.long()
    total = int(counts.sum())
    rows = torch.repeat_interleave(torch.arange(counts.numel(), device=counts.device), counts, output_size=total)
    first = torch.cumsum(counts, 0) - counts
    within = torch.arange(total, device=counts.device) - first[rows]
    return starts.long()[rows] + within, rows


def _range_sum(values: torch.Tensor, starts: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Sum of ``values[s : s + c]`` for every range, via an fp64 prefix sum (rows may be vectors)."""
    flat = values.reshape(values.shape[0], -1).double()
    prefix = torch.cat([flat.new_zeros(1, flat.shape[1]), torch.cumsum(flat, 0)], 0)
    out = prefix[starts + counts] - prefix[starts]
    return out.reshape((starts.numel(),) + values.shape[1:])


@dataclass
class NodeAggregates:
    """Per-node weighted centroid and weighted mean of every per-point feature."""

    centroid: torch.Tensor
    data: Dict[str, torch.Tensor]


@dataclass
class InteractionPlan:
    """Flat interaction lists of one (targets, sources) pair of trees."""

    near_targets: torch.Tensor
    near_sources: torch.Tensor
    far_targets: torch.Tensor
    far_nodes: torch.Tensor

    @property
    def n_near(self) -> int:
        return int(self.near_targets.numel())

    @property
    def n_far(self) -> int:
        return int(self.far_targets.numel())

    def to(self, device) -> "InteractionPlan":
        return InteractionPlan(*(t.to(device) for t in (self.near_targets, self.near_sources, self.far_targets, self.far_nodes)))


class ClusterTree:
    """Balanced binary tree over points; node ``i`` owns ``order[start[i] : start[i] + count[i]]``.

    ``left`` / ``right`` hold child node ids (``-1`` at a leaf), ``lo`` / ``hi`` the axis-aligned
    boxes and ``diag`` their diagonals.  Node 0 is the root; children always have larger ids than
    their parent.
    """

    def __init__(self, order, start, count, left, right, lo, hi, leaf_size: int):
        self.order, self.start, self.count = order, start, count
        self.left, self.right, self.lo, self.hi = left, right, lo, hi
        self.diag = torch.linalg.norm(hi - lo, dim=1) if lo.numel() else lo.new_zeros(0)
        self.leaf_size = leaf_size

    @property
    def n_nodes(self) -> int:
        return int(self.start.numel())

    @property
    def n_points(self) -> int:
        return int(self.order.numel())

    @property
    def device(self):
        return self.order.device

    def to(self, device) -> "ClusterTree":
        t = ClusterTree.__new__(ClusterTree)
        for k, v in self.__dict__.items():
            setattr(t, k, v.to(device) if isinstance(v, torch.Tensor) else v)
        return t

    # ------------------------------------------------------------------ build
    @classmethod
    def from_points(cls, points: torch.Tensor, leaf_size: int = 1) -> "ClusterTree":
        if points.ndim != 2:
            raise ValueError(f"points must have shape (n, d), got {tuple(points.shape)}")
        if leaf_size < 1:
            raise ValueError(f"leaf_size must be at least 1, got {leaf_size}")
        n, d = points.shape
        dev = points.device
        L = dict(dtype=torch.long, device=dev)
        if n == 0:
            e = torch.empty(0, **L)
            return cls(e, e, e, e, e, points.new_empty(0, d), points.new_empty(0, d), leaf_size)
        pts = points.detach()
        order = torch.arange(n, **L)
        starts, counts = [torch.zeros(1, **L)], [torch.full((1,), n, **L)]
        links = []                                   # (parent ids, left ids, right ids) per level
        act_id, act_start, act_count = torch.zeros(1, **L), starts[0], counts[0]
        n_nodes = 1
        while True:
            big = act_count > leaf_size
            ids, s, c = act_id[big], act_start[big], act_count[big]
            k = int(ids.numel())
            if k == 0:
                break
            pos, seg = ragged_arange(s, c)
            p = pts[order[pos]]
            seg_d = seg[:, None].expand(-1, d)
            lo = p.new_full((k, d), float("inf")).scatter_reduce_(0, seg_d, p, "amin")
            hi = p.new_full((k, d), float("-inf")).scatter_reduce_(0, seg_d, p, "amax")
            axis = (hi - lo).argmax(1)
            coord = p.gather(1, axis[seg][:, None]).squeeze(1)
            by_coord = torch.argsort(coord, stable=True)
            perm = by_coord[torch.argsort(seg[by_coord], stable=True)]   # grouped by node, sorted inside
            order[pos] = order[pos][perm]
            c_left = (c + 1) // 2
            lid = n_nodes + 2 * torch.arange(k, **L)
            links.append((ids, lid, lid + 1))
            act_id = torch.stack([lid, lid + 1], 1).reshape(-1)
            act_start = torch.stack([s, s + c_left], 1).reshape(-1)
            act_count = torch.stack([c_left, c - c_left], 1).reshape(-1)
            starts.append(act_start)
            counts.append(act_count)
            n_nodes += 2 * k
        start, count = torch.cat(starts), torch.cat(counts)
        left = torch.full((n_nodes,), -1, **L)
        right = torch.full((n_nodes,), -1, **L)
        for ids, lid, rid in links:
            left[ids], right[ids] = lid, rid
        # boxes: leaves from their points, inner nodes from their children (deepest level first)
        lo = pts.new_full((n_nodes, d), float("inf"))
        hi = pts.new_full((n_nodes, d), float("-inf"))
        leaf = (left < 0).nonzero().squeeze(1)
        pos, seg = ragged_arange(start[leaf], count[leaf])
        p = pts[order[pos]]
        tgt = leaf[seg][:, None].expand(-1, d)
        lo.scatter_reduce_(0, tgt, p, "amin")
        hi.scatter_reduce_(0, tgt, p, "amax")
        for ids, lid, rid in reversed(links):
            lo[ids] = torch.minimum(lo[lid], lo[rid])
            hi[ids] = torch.maximum(hi[lid], hi[rid])
        return cls(order, start, count, left, right, lo, hi, leaf_size)

    # ------------------------------------------------------------- node sums
    def node_sums(self, values: torch.Tensor) -> torch.Tensor:
        """Sum of a per-point quantity over every node (differentiable in ``values``)."""
        if self.n_nodes == 0:
            return values.new_zeros((0,) + values.shape[1:])
        return _range_sum(values[self.order], self.start, self.count).to(values.dtype)

    def aggregates(self, points: torch.Tensor, weights: Optional[torch.Tensor] = None,
                   data: Optional[Mapping[str, torch.Tensor]] = None) -> NodeAggregates:
        """Weighted centroid and weighted feature means per node; nodes of zero total weight give zeros."""
        if weights is None:
            weights = points.new_ones(points.shape[0])
        total = self.node_sums(weights.double())
        ok = total != 0
        safe = torch.where(ok, total, torch.ones_like(total))

        def mean(t: torch.Tensor) -> torch.Tensor:
            w = weights.reshape((-1,) + (1,) * (t.ndim - 1))
            s = self.node_sums((t * w).double())
            shape = (-1,) + (1,) * (t.ndim - 1)
            return torch.where(ok.reshape(shape), s / safe.reshape(shape), torch.zeros_like(s)).to(t.dtype)

        return NodeAggregates(mean(points), {k: mean(v) for k, v in dict(data or {}).items()})

    # -------------------------------------------------------------- traversal
    def find_interactions(self, target_tree: "ClusterTree", theta: float = 1.0) -> InteractionPlan:
        """Interaction lists between the points of ``target_tree`` and the sources of this tree.

        A (target node, source node) pair is *far* when ``(D_T + D_S) / r < theta`` with the box
        diagonals ``D`` and the smallest distance ``r`` between the two boxes; ``theta = 0`` makes
        every interaction exact.  Every (target, source) combination is covered exactly once, either
        by a near pair or through one far node that contains the source.
        """
        if theta < 0:
            raise ValueError(f"theta must be non-negative, got {theta}")
        S, T = self, target_tree
        dev = S.device
        L = dict(dtype=torch.long, device=dev)
        near_t, near_s, far_t, far_n = [], [], [], []
        if S.n_nodes and T.n_nodes:
            ft, fs = torch.zeros(1, **L), torch.zeros(1, **L)
        else:
            ft = fs = torch.empty(0, **L)
        while ft.numel():
            gap = torch.maximum(T.lo[ft] - S.hi[fs], S.lo[fs] - T.hi[ft]).clamp_min(0)
            r = torch.linalg.norm(gap, dim=1)
            far = (T.diag[ft] + S.diag[fs]) < theta * r
            t_leaf, s_leaf = T.left[ft] < 0, S.left[fs] < 0
            near = ~far & t_leaf & s_leaf
            if bool(far.any()):
                tn, sn = ft[far], fs[far]
                pos, row = ragged_arange(T.start[tn], T.count[tn])
                far_t.append(T.order[pos])
                far_n.append(sn[row])
            if bool(near.any()):
                tn, sn = ft[near], fs[near]
                ct, cs = T.count[tn], S.count[sn]
                idx, row = ragged_arange(torch.zeros_like(ct), ct * cs)
                near_t.append(T.order[T.start[tn][row] + idx // cs[row]])
                near_s.append(S.order[S.start[sn][row] + idx % cs[row]])
            rest = ~far & ~near
            tn, sn = ft[rest], fs[rest]
            tl, sl = t_leaf[rest], s_leaf[rest]
            split_t = ~tl & (sl | (T.diag[tn] >= S.diag[sn]))
            a_t, a_s = tn[split_t], sn[split_t]
            b_t, b_s = tn[~split_t], sn[~split_t]
            ft = torch.cat([T.left[a_t], T.right[a_t], b_t, b_t])
            fs = torch.cat([a_s, a_s, S.left[b_s], S.right[b_s]])

        def cat(parts):
            return torch.cat(parts) if parts else torch.empty(0, **L)

        return InteractionPlan(cat(near_t), cat(near_s), cat(far_t), cat(far_n))
