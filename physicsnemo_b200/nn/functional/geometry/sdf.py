"""Signed distance to a triangle surface, and ray–mesh intersection.

Parity: ``physicsnemo/nn/functional/geometry/sdf.py`` (``signed_distance_field`` → (signed distance, hit point, hit
face); NaN / −1 beyond ``max_dist``; sign from the hit face's normal or, with ``use_sign_winding_number``, from the
generalised winding number, which tolerates open or self-intersecting surfaces) and
``ray_mesh_intersect/ray_mesh_intersect.py`` (→ hit mask, distance, point, face id, geometric normal).

``"cuda"``: stack traversal of the implicit BVH of ``physicsnemo_b200.mesh.spatial.BVH`` (``csrc/bvh.cu``); the
hierarchy is built with tensor operations and can be passed back in (``bvh=``) for repeated queries of a static
mesh.  ``"torch"``: chunked all-pairs evaluation (CPU path and oracle).
"""
from __future__ import annotations

import ctypes

import torch

from ....core.function_spec import FunctionSpec
from ....ops import _lib
from ....ops import gemm as _g


def _faces(mesh_vertices, mesh_indices):
    if mesh_indices.ndim == 2:
        if mesh_indices.shape[-1] != 3:
            raise ValueError("mesh_indices with 2 dimensions must have shape (n_faces, 3)")
    elif mesh_indices.ndim == 1:
        if mesh_indices.numel() == 0 or mesh_indices.numel() % 3:
            raise ValueError("mesh_indices must contain complete triangle faces")
        mesh_indices = mesh_indices.reshape(-1, 3)
    else:
        raise ValueError("mesh_indices must be either 1D flattened indices or 2D (n_faces, 3)")
    if mesh_indices.numel() == 0:
        raise ValueError("mesh_indices must contain complete triangle faces")
    if not mesh_indices.is_cuda:
        lo, hi = int(mesh_indices.min()), int(mesh_indices.max())
        if lo < 0 or hi >= mesh_vertices.shape[0]:
            raise ValueError(f"mesh_indices must index existing vertices; got range [{lo}, {hi}] for {mesh_vertices.shape[0]} vertices")
    return mesh_indices.long()


def _sign(vertices, faces, pts, cp, face, use_winding, winding_fn):
    if use_winding:
        inside = winding_fn() > 0.5
    else:
        tri = vertices[faces[face.clamp_min(0)]]
        n = torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])
        inside = ((pts - cp) * n).sum(-1) < 0
    return torch.where(inside, -1.0, 1.0).to(pts.dtype)


def _sdf_torch(mesh_vertices, mesh_indices, input_points, max_dist: float = 1e8, use_sign_winding_number: bool = False):
    from ....mesh.spatial import closest_point_bruteforce, winding_number

    if input_points.shape[-1] != 3:
        raise ValueError("input_points must have last dimension of size 3")
    faces = _faces(mesh_vertices, mesh_indices)
    shape, dt = input_points.shape, input_points.dtype
    pts = input_points.reshape(-1, 3).float()
    v = mesh_vertices.float()
    if pts.shape[0] == 0:
        return pts.new_empty(shape[:-1]).to(dt), pts.new_empty(shape).to(dt), torch.empty(shape[:-1], dtype=torch.int64, device=pts.device)
    d, cp, face = closest_point_bruteforce(v, faces, pts)
    sgn = _sign(v, faces, pts, cp, face, use_sign_winding_number,
                lambda: torch.cat([winding_number(pts[s:s + 2048], v[faces]) for s in range(0, pts.shape[0], 2048)]))
    far = d > max_dist
    nan = torch.full_like(d, float("nan"))
    sdf = torch.where(far, nan, d * sgn)
    cp = torch.where(far[:, None], nan[:, None].expand(-1, 3), cp)
    face = torch.where(far, torch.full_like(face, -1), face)
    return sdf.reshape(shape[:-1]).to(dt), cp.reshape(shape).to(dt), face.reshape(shape[:-1])


def _lib_bvh():
    lib = _lib.load(required=True)
    if not getattr(lib, "_bvh_declared", False):
        c = ctypes
        vp = c.c_void_p
        lib.pnm_bvh_closest.argtypes = [vp] * 7 + [c.c_int, c.c_longlong, c.c_float, vp]
        lib.pnm_bvh_raycast.argtypes = [vp] * 8 + [c.c_int, c.c_longlong, c.c_float, vp]
        lib.pnm_winding_number.argtypes = [vp, vp, vp, c.c_longlong, c.c_longlong, vp]
        for f in (lib.pnm_bvh_closest, lib.pnm_bvh_raycast, lib.pnm_winding_number):
            f.restype = c.c_int
        lib._bvh_declared = True
    return lib


def _sdf_cuda(mesh_vertices, mesh_indices, input_points, max_dist: float = 1e8, use_sign_winding_number: bool = False, bvh=None):
    from ....mesh.spatial import BVH

    if input_points.shape[-1] != 3:
        raise ValueError("input_points must have last dimension of size 3")
    faces = _faces(mesh_vertices, mesh_indices)
    shape, dt = input_points.shape, input_points.dtype
    pts = input_points.reshape(-1, 3).detach().float().contiguous()
    v = mesh_vertices.detach().float().contiguous()
    N = pts.shape[0]
    dist = torch.empty(N, dtype=torch.float32, device=pts.device)
    cp = torch.empty(N, 3, dtype=torch.float32, device=pts.device)
    face = torch.empty(N, dtype=torch.int64, device=pts.device)
    if N:
        lib = _lib_bvh()
        bvh = bvh if bvh is not None else BVH(v, faces)
        st = torch.cuda.current_stream().cuda_stream
        err = lib.pnm_bvh_closest(bvh.bounds.data_ptr(), bvh.order.data_ptr(), bvh.triangles.data_ptr(), pts.data_ptr(),
                                  dist.data_ptr(), cp.data_ptr(), face.data_ptr(), bvh.n_leaves, N, min(float(max_dist), 1e18), st)
        if err:
            raise RuntimeError(f"pnm_bvh_closest failed ({err})")
        _g.launch_count += 1

        def wn():
            out = torch.empty(N, dtype=torch.float32, device=pts.device)
            e = lib.pnm_winding_number(bvh.triangles.data_ptr(), pts.data_ptr(), out.data_ptr(), bvh.n_faces, N, st)
            if e:
                raise RuntimeError(f"pnm_winding_number failed ({e})")
            _g.launch_count += 1
            return out

        dist = dist * _sign(v, faces, pts, torch.nan_to_num(cp), face, use_sign_winding_number, wn)
    return dist.reshape(shape[:-1]).to(dt), cp.reshape(shape).to(dt), face.reshape(shape[:-1])


def _winding_cuda(vertices, faces, pts):
    """Generalized winding number of ``pts [N, 3]`` (exact sum of signed solid angles over all faces) on the GPU."""
    lib = _lib_bvh()
    tri = vertices.detach().float()[faces].contiguous()
    pts = pts.detach().float().contiguous()
    out = torch.empty(pts.shape[0], dtype=torch.float32, device=pts.device)
    if pts.shape[0]:
        e = lib.pnm_winding_number(tri.data_ptr(), pts.data_ptr(), out.data_ptr(), tri.shape[0], pts.shape[0],
                                   torch.cuda.current_stream().cuda_stream)
        if e:
            raise RuntimeError(f"pnm_winding_number failed ({e})")
        _g.launch_count += 1
    return out


class SignedDistanceField(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(mesh_vertices, mesh_indices, input_points, max_dist=1e8, use_sign_winding_number=False, bvh=None):
        return _sdf_cuda(mesh_vertices, mesh_indices, input_points, max_dist, use_sign_winding_number, bvh)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(mesh_vertices, mesh_indices, input_points, max_dist=1e8, use_sign_winding_number=False, bvh=None):
        return _sdf_torch(mesh_vertices, mesh_indices, input_points, max_dist, use_sign_winding_number)


def _ray_finish(v, faces, o, d, t, face, shape):
    hit = face >= 0
    dn = d / d.norm(dim=-1, keepdim=True).clamp_min(1e-30)
    pts = torch.where(hit[:, None], o + dn * torch.where(hit, t, torch.zeros_like(t))[:, None], torch.zeros_like(o))
    tri = v[faces[face.clamp_min(0)]]
    n = torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])
    n = n / n.norm(dim=-1, keepdim=True).clamp_min(1e-30)
    n = torch.where(hit[:, None], n, torch.zeros_like(n))
    t = torch.where(hit, t, torch.full_like(t, float("inf")))
    return hit.reshape(shape[:-1]), t.reshape(shape[:-1]), pts.reshape(shape), face.reshape(shape[:-1]), n.reshape(shape)


def _ray_torch(mesh_vertices, mesh_indices, ray_origins, ray_directions, max_distance: float = 1.0e8, bvh=None, return_bvh=False):
    from ....mesh.spatial import ray_triangle_bruteforce

    faces = _faces(mesh_vertices, mesh_indices)
    shape = ray_origins.shape
    o, d = ray_origins.reshape(-1, 3).float(), ray_directions.reshape(-1, 3).float()
    v = mesh_vertices.float()
    dn = d / d.norm(dim=-1, keepdim=True).clamp_min(1e-30)
    t, face, _, _ = ray_triangle_bruteforce(v, faces, o, dn)
    face = torch.where(t <= max_distance, face, torch.full_like(face, -1))
    out = _ray_finish(v, faces, o, d, t, face, shape)
    return (*out, None) if return_bvh else out


def _ray_cuda(mesh_vertices, mesh_indices, ray_origins, ray_directions, max_distance: float = 1.0e8, bvh=None, return_bvh=False):
    from ....mesh.spatial import BVH

    faces = _faces(mesh_vertices, mesh_indices)
    shape = ray_origins.shape
    o = ray_origins.reshape(-1, 3).detach().float().contiguous()
    d = ray_directions.reshape(-1, 3).detach().float().contiguous()
    v = mesh_vertices.detach().float().contiguous()
    N = o.shape[0]
    t = torch.empty(N, dtype=torch.float32, device=o.device)
    face = torch.empty(N, dtype=torch.int64, device=o.device)
    uv = torch.empty(N, 2, dtype=torch.float32, device=o.device)
    bvh = bvh if bvh is not None else BVH(v, faces)
    if N:
        lib = _lib_bvh()
        err = lib.pnm_bvh_raycast(bvh.bounds.data_ptr(), bvh.order.data_ptr(), bvh.triangles.data_ptr(), o.data_ptr(), d.data_ptr(),
                                  t.data_ptr(), face.data_ptr(), uv.data_ptr(), bvh.n_leaves, N, min(float(max_distance), 1e30),
                                  torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_bvh_raycast failed ({err})")
        _g.launch_count += 1
    out = _ray_finish(v, faces, o, d, t, face, shape)
    return (*out, bvh) if return_bvh else out


class RayMeshIntersect(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(mesh_vertices, mesh_indices, ray_origins, ray_directions, max_distance=1.0e8, bvh=None, return_bvh=False):
        return _ray_cuda(mesh_vertices, mesh_indices, ray_origins, ray_directions, max_distance, bvh, return_bvh)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(mesh_vertices, mesh_indices, ray_origins, ray_directions, max_distance=1.0e8, bvh=None, return_bvh=False):
        return _ray_torch(mesh_vertices, mesh_indices, ray_origins, ray_directions, max_distance, bvh, return_bvh)


signed_distance_field = SignedDistanceField.make_function("signed_distance_field")
ray_mesh_intersect = RayMeshIntersect.make_function("ray_mesh_intersect")
