"""Hierarchy of named process groups.

Parity: ``physicsnemo/distributed/config.py`` (``ProcessGroupNode``, ``ProcessGroupConfig`` with
``add_node``, ``leaf_groups``, ``set_leaf_group_sizes``, ``update_parent_sizes``).  The reference
stores the hierarchy in a ``treelib.Tree``; here a small tree class with the same accessors
(``children``, ``get_node``, ``leaves``, ``parent``, ``show``) removes that dependency.
"""
from __future__ import annotations

from typing import Dict, List, Optional


class ProcessGroupNode:
    """Node of the group hierarchy: ``name`` and (once known) ``size``."""

    def __init__(self, name: str, size: Optional[int] = None):
        self.name = name
        self.size = size

    def __str__(self):
        return f"ProcessGroupNode(name={self.name}, size={self.size}, "

    def __repr__(self):
        return self.__str__()


class _TreeNode:
    def __init__(self, identifier: str, data: ProcessGroupNode, parent: Optional[str]):
        self.identifier = identifier
        self.tag = identifier
        self.data = data
        self.parent_id = parent
        self.child_ids: List[str] = []

    def is_leaf(self):
        return not self.child_ids


class _Tree:
    """Minimal ordered tree keyed by node identifier."""

    def __init__(self):
        self.nodes: Dict[str, _TreeNode] = {}
        self.root: Optional[str] = None

    def create_node(self, tag, identifier, data=None, parent=None):
        if identifier in self.nodes:
            raise ValueError(f"Node with name {identifier} already exists")
        if parent is None:
            if self.root is not None:
                raise ValueError("Tree already has a root")
            self.root = identifier
        else:
            if parent not in self.nodes:
                raise ValueError(f"Parent {parent} does not exist")
            self.nodes[parent].child_ids.append(identifier)
        node = _TreeNode(identifier, data, parent)
        self.nodes[identifier] = node
        return node

    def get_node(self, identifier):
        return self.nodes.get(identifier)

    def children(self, identifier):
        return [self.nodes[c] for c in self.nodes[identifier].child_ids]

    def parent(self, identifier):
        p = self.nodes[identifier].parent_id
        return None if p is None else self.nodes[p]

    def leaves(self):
        return [n for n in self.nodes.values() if n.is_leaf()]

    def expand_tree(self, mode="bfs"):
        order, frontier = [], [self.root]
        while frontier:
            nid = frontier.pop(0)
            order.append(nid)
            frontier.extend(self.nodes[nid].child_ids)
        return order

    def show(self, indent: int = 0, nid=None):
        nid = self.root if nid is None else nid
        lines = ["  " * indent + nid]
        for c in self.nodes[nid].child_ids:
            lines.append(self.show(indent + 1, c))
        return "\n".join(lines)

    def __str__(self):
        return self.show()


class ProcessGroupConfig:
    """Tree of ``ProcessGroupNode``; leaf sizes determine every parent's size (their product)."""

    def __init__(self, node: ProcessGroupNode):
        self.root = node
        self.root_id = node.name
        self.tree = _Tree()
        self.tree.create_node(node.name, node.name, data=node)

    def add_node(self, node: ProcessGroupNode, parent=Optional[str]):
        if isinstance(parent, ProcessGroupNode):
            parent = parent.name
        if not isinstance(parent, str):
            raise ValueError("A parent node (name or ProcessGroupNode) is required")
        self.tree.create_node(node.name, node.name, data=node, parent=parent)

    def get_node(self, name: str) -> ProcessGroupNode:
        return self.tree.get_node(name).data

    def update_parent_sizes(self, verbose: bool = False) -> int:
        return self._tree_product_reduction(self.tree, self.root_id, verbose=verbose)

    def leaf_groups(self) -> List[str]:
        return [n.identifier for n in self.tree.leaves()]

    def set_leaf_group_sizes(self, group_sizes: Dict[str, int], update_parent_sizes: bool = True):
        for name, size in group_sizes.items():
            node = self.tree.get_node(name)
            if node is None or not node.is_leaf():
                raise AssertionError(f"Group {name} is not a leaf group")
            node.data.size = size
        if update_parent_sizes:
            self.update_parent_sizes()

    @staticmethod
    def _tree_product_reduction(tree, node_id, verbose=False):
        children = tree.children(node_id)
        node = tree.get_node(node_id)
        if not children:
            if node.data.size is None:
                raise AssertionError("Leaf nodes should have a valid size set")
            return node.data.size
        product = 1
        for child in children:
            product *= ProcessGroupConfig._tree_product_reduction(tree, child.identifier, verbose)
        node.data.size = product
        if verbose:
            print(node.data)
        return product
