"""Hierarchy of icosahedral meshes on the unit sphere.

Parity: ``physicsnemo/models/graphcast/utils/icosahedral_mesh.py`` (``TriangularMesh``,
``get_icosahedron``, ``get_hierarchy_of_triangular_meshes_for_sphere``, ``merge_meshes``,
``faces_to_edges``).  The icosahedron has the reference's vertex order and orientation (two faces
symmetric about the x–z plane after a rotation about y), its faces are found geometrically
(mutually adjacent vertex triples, oriented outward); every refinement splits each triangle in four,
with the new vertices numbered after the old ones in order of first use, so coarse meshes are
prefixes of fine ones.  Refinement is an array computation (unique edge keys), not a Python loop
over faces.
"""
from __future__ import annotations

import itertools
from typing import List, NamedTuple, Sequence, Tuple

import numpy as np


class TriangularMesh(NamedTuple):
    vertices: np.ndarray
    faces: np.ndarray


def get_icosahedron() -> TriangularMesh:
    phi = (1 + np.sqrt(5)) / 2
    verts = []
    for c1 in (1.0, -1.0):
        for c2 in (phi, -phi):
            verts += [(c1, c2, 0.0), (0.0, c1, c2), (c2, 0.0, c1)]
    v = np.array(verts, dtype=np.float32)
    v /= np.linalg.norm([1.0, phi])
    # faces: triples of mutually nearest vertices (edge length 2 / |(1, phi)|), counter-clockwise seen from outside
    d = np.linalg.norm(v[:, None] - v[None], axis=-1)
    edge = np.isclose(d, d[d > 1e-6].min(), rtol=1e-4)
    faces = []
    for a, b, c in itertools.combinations(range(12), 3):
        if edge[a, b] and edge[b, c] and edge[a, c]:
            if np.dot(np.cross(v[b] - v[a], v[c] - v[a]), v[a] + v[b] + v[c]) < 0:
                b, c = c, b
            faces.append((a, b, c))
    angle_between_faces = 2 * np.arcsin(phi / np.sqrt(3))
    a = (np.pi - angle_between_faces) / 2
    rot_y = np.array([[np.cos(a), 0.0, np.sin(a)], [0.0, 1.0, 0.0], [-np.sin(a), 0.0, np.cos(a)]])
    return TriangularMesh(vertices=np.dot(v, rot_y).astype(np.float32), faces=np.array(faces, dtype=np.int32))


def _two_split_unit_sphere_triangle_faces(mesh: TriangularMesh) -> TriangularMesh:
    f = mesh.faces.astype(np.int64)
    n = mesh.vertices.shape[0]
    # per face, the edges (1,2), (2,3), (3,1) in that order; one midpoint per undirected edge
    pairs = np.stack([f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]], axis=1).reshape(-1, 2)
    key = np.sort(pairs, axis=1)
    key = key[:, 0] * n + key[:, 1]
    uniq, first, inverse = np.unique(key, return_index=True, return_inverse=True)
    order = np.argsort(first, kind="stable")                  # number midpoints by first use
    rank = np.empty_like(order)
    rank[order] = np.arange(order.size)
    mid_index = (n + rank[inverse]).reshape(-1, 3)            # [F, 3]: m12, m23, m31
    lo, hi = uniq[order] // n, uniq[order] % n
    parents = mesh.vertices.astype(np.float32)
    mids = (parents[lo] + parents[hi]) / 2
    mids /= np.linalg.norm(mids, axis=1, keepdims=True)
    m12, m23, m31 = mid_index[:, 0], mid_index[:, 1], mid_index[:, 2]
    new_faces = np.stack([np.stack([f[:, 0], m12, m31], 1), np.stack([m12, f[:, 1], m23], 1),
                          np.stack([m31, m23, f[:, 2]], 1), np.stack([m12, m23, m31], 1)], axis=1).reshape(-1, 3)
    return TriangularMesh(vertices=np.concatenate([parents, mids.astype(np.float32)], 0), faces=new_faces.astype(np.int32))


def get_hierarchy_of_triangular_meshes_for_sphere(splits: int) -> List[TriangularMesh]:
    meshes = [get_icosahedron()]
    for _ in range(splits):
        meshes.append(_two_split_unit_sphere_triangle_faces(meshes[-1]))
    return meshes


def merge_meshes(mesh_list: Sequence[TriangularMesh]) -> TriangularMesh:
    """Finest vertices with the faces of all levels (the "multimesh")."""
    for coarse, fine in itertools.pairwise(mesh_list):
        k = coarse.vertices.shape[0]
        if not np.allclose(coarse.vertices, fine.vertices[:k]):
            raise ValueError("meshes are not nested: coarse vertices must be a prefix of the finer mesh")
    return TriangularMesh(vertices=mesh_list[-1].vertices, faces=np.concatenate([m.faces for m in mesh_list], axis=0))


def faces_to_edges(faces: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    if faces.ndim != 2 or faces.shape[-1] != 3:
        raise ValueError("faces must have shape (F, 3)")
    return (np.concatenate([faces[:, 0], faces[:, 1], faces[:, 2]]), np.concatenate([faces[:, 1], faces[:, 2], faces[:, 0]]))
