"""Dependency scheduler that turns a bag of ``Computation`` nodes into an ordered ``nn.Module``.

Parity: ``physicsnemo/sym/graph.py`` (``Graph``): prune the nodes to those the requested names
depend on, emit every node whose inputs are available, and whenever the remaining nodes are
blocked on derivative keys, emit the gradient nodes that produce them.  The schedule is computed
once at construction; ``forward`` walks a ``ModuleList``.

The scheduler here is a worklist over name sets (each pass scans an immutable snapshot), so a
node is never skipped because its predecessor was removed from the list being iterated.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from .computation import Computation
from .constants import diff_str


def _base(name: str) -> str:
    return name.split(diff_str)[0]


def _computable_names(nodes: Sequence[Computation], invar: Sequence[str]) -> List[str]:
    """Names reachable from ``invar`` ignoring derivative requirements."""
    names, pending = list(invar), list(nodes)
    progressed = True
    while progressed:
        progressed = False
        have = set(names)
        rest = []
        for node in pending:
            if set(node.inputs) <= have:
                names += node.outputs
                have.update(node.outputs)
                progressed = True
            else:
                rest.append(node)
        pending = rest
    return names


def _prune_nodes(nodes: Sequence[Computation], req_names: Sequence[str]) -> List[Computation]:
    """Nodes that (transitively) feed the requested names."""
    wanted = set(req_names) | {_base(n) for n in req_names}
    kept, pending = [], list(nodes)
    progressed = True
    while progressed:
        progressed = False
        rest = []
        for node in pending:
            if wanted & set(node.outputs):
                wanted.update(node.inputs)
                wanted.update(node.derivatives)
                wanted.update(_base(d) for d in node.derivatives)
                kept.append(node)
                progressed = True
            else:
                rest.append(node)
        pending = rest
    return kept


def _collect_needed_derivatives(remaining: Sequence[Computation], req_names: Sequence[str]) -> List[str]:
    out: List[str] = []
    for node in remaining:
        out += node.derivatives
    return out + [n for n in req_names if diff_str in n]


def _print_graph_unroll_error(nodes, invar, req_names) -> None:
    bar = "=" * 60
    print(bar)
    print("Could not unroll graph!")
    print(f"  invar: {invar}")
    print(f"  requested: {req_names}")
    print(f"  computable: {_computable_names(nodes, invar)}")
    for node in nodes:
        print(f"  node: {node}")
    print(bar)


class Graph(torch.nn.Module):
    def __init__(self, nodes: List[Computation], invar: List[str], req_names: List[str],
                 diff_nodes: List[Computation] | None = None):
        super().__init__()
        diff_nodes = list(diff_nodes or [])
        self.req_names = list(req_names)
        if not {_base(n) for n in req_names} <= set(_computable_names(nodes, invar)):
            _print_graph_unroll_error(nodes, invar, req_names)
            raise RuntimeError("Failed unrolling graph")
        pending = _prune_nodes(nodes, req_names)
        order: List[Computation] = []
        have = list(invar)
        while True:
            before = len(have)
            progressed = True
            while progressed:
                progressed = False
                avail, rest = set(have), []
                for node in pending:
                    if set(node.inputs + node.derivatives) <= avail:
                        order.append(node)
                        have += node.outputs
                        avail.update(node.outputs)
                        progressed = True
                    else:
                        rest.append(node)
                pending = rest
            missing = [d for d in _collect_needed_derivatives(pending, req_names) if d not in have]
            if missing:
                for dn in diff_nodes:
                    if set(dn.outputs) & set(missing) and set(dn.inputs) <= set(have) and dn not in order:
                        order.append(dn)
                        have += dn.outputs
            if set(req_names) <= set(have):
                break
            if len(have) == before:
                raise RuntimeError(
                    f"Graph scheduler stalled — cannot satisfy: {set(req_names) - set(have)}. "
                    f"Available: {sorted(set(have))}. Remaining nodes: {[str(n) for n in pending]}")
        self.node_evaluation_order = order
        self.evaluation_order = torch.nn.ModuleList([n.evaluate for n in order])
        self.node_names: List[str] = [n.name for n in order]

    def forward(self, invar: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        values = dict(invar)
        for module in self.evaluation_order:
            values.update(module(values))
        return {k: v for k, v in values.items() if k in self.req_names}
