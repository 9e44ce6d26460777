"""Mesh file IO: native OBJ / ASCII-or-binary STL readers and writers, and pyvista conversion when pyvista exists
(parity: ``physicsnemo/mesh/io``)."""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np
import torch

from .mesh import Mesh


def read_obj(path) -> Mesh:
    pts, polys = [], []
    with open(path) as f:
        for line in f:
            tok = line.split()
            if not tok:
                continue
            if tok[0] == "v":
                pts.append([float(x) for x in tok[1:4]])
            elif tok[0] == "f":
                ids = [int(t.split("/")[0]) for t in tok[1:]]
                polys.append([i - 1 if i > 0 else len(pts) + i for i in ids])
    return Mesh.from_polygons(torch.tensor(pts, dtype=torch.float32), polys)


def write_obj(mesh: Mesh, path) -> None:
    if mesh.n_manifold_dims != 2:
        raise ValueError("OBJ export needs a triangle mesh")
    p = mesh.points.detach().cpu()
    if p.shape[1] == 2:
        p = torch.nn.functional.pad(p, (0, 1))
    with open(path, "w") as f:
        f.writelines(f"v {x:.9g} {y:.9g} {z:.9g}\n" for x, y, z in p.tolist())
        f.writelines(f"f {a + 1} {b + 1} {c + 1}\n" for a, b, c in mesh.cells.cpu().tolist())


def read_stl(path) -> Mesh:
    raw = Path(path).read_bytes()
    if raw[:5].lower() == b"solid" and b"facet" in raw[:1000]:
        vals = [[float(x) for x in ln.split()[1:4]] for ln in raw.decode(errors="ignore").splitlines() if ln.strip().startswith("vertex")]
        tri = np.asarray(vals, dtype=np.float32).reshape(-1, 3, 3)
    else:
        n = struct.unpack("<I", raw[80:84])[0]
        rec = np.frombuffer(raw, dtype=np.dtype([("n", "<f4", 3), ("v", "<f4", (3, 3)), ("a", "<u2")]), count=n, offset=84)
        tri = rec["v"].copy()
    pts = torch.from_numpy(tri.reshape(-1, 3))
    cells = torch.arange(pts.shape[0]).reshape(-1, 3)
    return Mesh(pts, cells).clean(tolerance=1e-9)


def write_stl(mesh: Mesh, path) -> None:
    if mesh.n_manifold_dims != 2 or mesh.n_spatial_dims != 3:
        raise ValueError("STL export needs a triangle mesh in 3-D")
    tri = mesh.points[mesh.cells].detach().cpu().numpy().astype("<f4")
    nrm = mesh.cell_normals.detach().cpu().numpy().astype("<f4")
    rec = np.zeros(tri.shape[0], dtype=np.dtype([("n", "<f4", 3), ("v", "<f4", (3, 3)), ("a", "<u2")]))
    rec["n"], rec["v"] = nrm, tri
    with open(path, "wb") as f:
        f.write(b"physicsnemo_b200 binary STL".ljust(80, b" "))
        f.write(struct.pack("<I", tri.shape[0]))
        f.write(rec.tobytes())


def from_pyvista(pv_mesh) -> Mesh:
    """``pyvista.PolyData`` / ``UnstructuredGrid`` (triangles or tetrahedra) → ``Mesh`` with its data arrays."""
    pts = torch.from_numpy(np.asarray(pv_mesh.points, dtype=np.float32))
    if hasattr(pv_mesh, "faces") and pv_mesh.faces.size:
        tri = pv_mesh.triangulate()
        cells = torch.from_numpy(np.asarray(tri.faces).reshape(-1, 4)[:, 1:].astype(np.int64))
    elif hasattr(pv_mesh, "cells_dict"):
        import pyvista as pv

        cells = torch.from_numpy(np.asarray(pv_mesh.cells_dict[pv.CellType.TETRA], dtype=np.int64))
    else:
        cells = None
    pd = {k: torch.from_numpy(np.asarray(pv_mesh.point_data[k])) for k in pv_mesh.point_data.keys()}
    cd = {k: torch.from_numpy(np.asarray(pv_mesh.cell_data[k])) for k in pv_mesh.cell_data.keys()} if cells is not None else {}
    cd = {k: v for k, v in cd.items() if cells is not None and v.shape[0] == cells.shape[0]}
    return Mesh(pts, cells, pd, cd)


def to_pyvista(mesh: Mesh):
    import pyvista as pv

    p = mesh.points.detach().cpu().numpy()
    if p.shape[1] == 2:
        p = np.pad(p, ((0, 0), (0, 1)))
    c = mesh.cells.cpu().numpy()
    if mesh.n_manifold_dims == 2:
        out = pv.PolyData(p, np.hstack([np.full((c.shape[0], 1), 3), c]).ravel())
    elif mesh.n_manifold_dims == 3:
        out = pv.UnstructuredGrid({pv.CellType.TETRA: c}, p)
    elif mesh.n_manifold_dims == 1:
        out = pv.PolyData(p, lines=np.hstack([np.full((c.shape[0], 1), 2), c]).ravel())
    else:
        out = pv.PolyData(p)
    for k, v in mesh.point_data.items():
        out.point_data[k] = v.detach().cpu().numpy()
    for k, v in mesh.cell_data.items():
        out.cell_data[k] = v.detach().cpu().numpy()
    return out


def read(path) -> Mesh:
    suffix = Path(path).suffix.lower()
    if suffix == ".obj":
        return read_obj(path)
    if suffix == ".stl":
        return read_stl(path)
    if suffix == ".pt":
        return Mesh.load(path)
    import pyvista as pv

    return from_pyvista(pv.read(str(path)))
