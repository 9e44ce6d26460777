"""Ray-cast rendering of triangle meshes.

Parity: ``physicsnemo/nn/functional/rendering/mesh_raycast`` (one primary ray per pixel, nearest
hit, geometric normal flipped toward the camera, uniform / per-vertex (barycentric) / per-face
colours, Lambert shading with an ambient floor; outputs RGBA, depth and normal images).

``"cuda"``: traversal of the implicit Morton BVH (``mesh.spatial.BVH``) and shading in one kernel
per image (``csrc/render.cu``); a prebuilt ``bvh`` can be passed to re-render a static mesh from
many cameras without rebuilding.  ``"torch"``: all-pairs ray / triangle tests; CPU path and oracle.
"""
from __future__ import annotations

import torch

from ....core.function_spec import FunctionSpec
from . import utils as U


def _prepare(mesh_vertices, mesh_indices, image_height, image_width, fov_y_degrees, vertex_colors, face_colors, surface_color,
             light_direction, ambient, max_distance, eye, center, up):
    if mesh_vertices.ndim != 2 or mesh_vertices.shape[-1] != 3:
        raise ValueError(f"mesh_vertices must have shape (num_vertices, 3), got {tuple(mesh_vertices.shape)}")
    if mesh_vertices.shape[0] == 0:
        raise ValueError("mesh_vertices must contain at least one vertex")
    if mesh_indices.ndim == 2:
        if mesh_indices.shape[-1] != 3:
            raise ValueError("mesh_indices must have shape (num_faces, 3)")
        mesh_indices = mesh_indices.reshape(-1)
    elif mesh_indices.ndim != 1:
        raise ValueError("mesh_indices must be 1D or have shape (num_faces, 3)")
    if mesh_indices.numel() == 0 or mesh_indices.numel() % 3 != 0:
        raise ValueError("mesh_indices must contain complete triangle faces")
    lo, hi = int(mesh_indices.min()), int(mesh_indices.max())
    if lo < 0 or hi >= mesh_vertices.shape[0]:
        raise ValueError(f"mesh_indices must index existing vertices; got range [{lo}, {hi}] for "
                         f"{mesh_vertices.shape[0]} vertices")
    if vertex_colors is not None and face_colors is not None:
        raise ValueError("Pass either vertex_colors or face_colors, not both")
    U.validate_image_shape(image_height, image_width)
    U.validate_fov(fov_y_degrees)
    U.validate_ambient(ambient)
    if max_distance <= 0.0:
        raise ValueError("max_distance must be strictly positive")
    dev = mesh_vertices.device
    faces = mesh_indices.to(device=dev, dtype=torch.int32).reshape(-1, 3).contiguous()
    mode, colors = 0, torch.zeros(1, 4, device=dev)
    if vertex_colors is not None:
        if vertex_colors.shape[0] != mesh_vertices.shape[0]:
            raise ValueError("vertex_colors must have one color per mesh vertex")
        mode, colors = 1, U.color_tensor(vertex_colors, device=dev, shape_name="vertex_colors", expected_rank=2)
    elif face_colors is not None:
        if face_colors.shape[0] != faces.shape[0]:
            raise ValueError("face_colors must have one color per mesh face")
        mode, colors = 2, U.color_tensor(face_colors, device=dev, shape_name="face_colors", expected_rank=2)
    return (mesh_vertices.to(torch.float32).contiguous(), faces, mode, colors, U.camera_basis(eye, center, up, device=dev),
            U.uniform_color_tensor(surface_color, device=dev), U.light_tensor(light_direction, device=dev))


def _cuda(mesh_vertices, mesh_indices, image_height, image_width, eye, center, up, fov_y_degrees, vertex_colors=None,
          face_colors=None, surface_color=None, light_direction=None, ambient=0.2, max_distance=1.0e8, bvh=None):
    from ....mesh.spatial import BVH

    v, faces, mode, colors, cam, uc, light = _prepare(mesh_vertices, mesh_indices, image_height, image_width, fov_y_degrees,
                                                      vertex_colors, face_colors, surface_color, light_direction, ambient,
                                                      max_distance, eye, center, up)
    dev = v.device
    bvh = bvh if bvh is not None else BVH(v, faces.long())
    rgba = torch.empty(image_height, image_width, 4, device=dev)
    depth = torch.empty(image_height, image_width, device=dev)
    normal = torch.empty(image_height, image_width, 3, device=dev)
    U.check(U.lib_render().pnm_mesh_raycast_render(
        bvh.bounds.data_ptr(), bvh.order.data_ptr(), bvh.triangles.data_ptr(), faces.data_ptr(), bvh.n_leaves,
        colors.data_ptr(), cam.data_ptr(), uc.data_ptr(), light.data_ptr(), image_width, image_height,
        U.tan_half(fov_y_degrees), image_width / image_height, min(float(max_distance), 1e30), float(ambient), mode,
        rgba.data_ptr(), depth.data_ptr(), normal.data_ptr(), U.stream()), "pnm_mesh_raycast_render")
    return rgba, U.finish_depth(depth), normal


def _torch(mesh_vertices, mesh_indices, image_height, image_width, eye, center, up, fov_y_degrees, vertex_colors=None,
           face_colors=None, surface_color=None, light_direction=None, ambient=0.2, max_distance=1.0e8, bvh=None):
    from ....mesh.spatial import ray_triangle_bruteforce

    v, faces, mode, colors, cam, uc, light = _prepare(mesh_vertices, mesh_indices, image_height, image_width, fov_y_degrees,
                                                      vertex_colors, face_colors, surface_color, light_direction, ambient,
                                                      max_distance, eye, center, up)
    dev, H, W = v.device, image_height, image_width
    d = U.pixel_rays(cam, H, W, fov_y_degrees)
    faces_l = faces.long()
    t, face, bu, bv = ray_triangle_bruteforce(v, faces_l, cam[0].expand_as(d), d)
    hit = (face >= 0) & (t <= max_distance)
    f = torch.where(hit, face, torch.zeros_like(face))
    tri = v[faces_l[f]]
    n = U.normalize(torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0]))
    n = torch.where(((n * d).sum(-1) > 0)[:, None], -n, n)
    if mode == 1:
        c = colors[faces_l[f]]
        color = (1 - bu - bv)[:, None] * c[:, 0] + bu[:, None] * c[:, 1] + bv[:, None] * c[:, 2]
    elif mode == 2:
        color = colors[f]
    else:
        color = uc.expand(H * W, 4)
    rgba = torch.where(hit[:, None], U.shade(color, n, light, ambient), torch.zeros(H * W, 4, device=dev))
    depth = torch.where(hit, t, torch.full_like(t, U.FAR))
    n = torch.where(hit[:, None], n, torch.zeros_like(n))
    return rgba.reshape(H, W, 4), U.finish_depth(depth.reshape(H, W)), n.reshape(H, W, 3)


class MeshRaycast(FunctionSpec):
    """``(rgba [H, W, 4], depth [H, W], normal [H, W, 3])`` of a triangle mesh seen from a pinhole camera."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(mesh_vertices, mesh_indices, image_height, image_width, eye, center, up, fov_y_degrees,
                     vertex_colors=None, face_colors=None, surface_color=None, light_direction=None, ambient=0.2,
                     max_distance=1.0e8, bvh=None):
        return _cuda(mesh_vertices, mesh_indices, image_height, image_width, eye, center, up, fov_y_degrees, vertex_colors,
                     face_colors, surface_color, light_direction, ambient, max_distance, bvh)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(mesh_vertices, mesh_indices, image_height, image_width, eye, center, up, fov_y_degrees,
                      vertex_colors=None, face_colors=None, surface_color=None, light_direction=None, ambient=0.2,
                      max_distance=1.0e8, bvh=None):
        return _torch(mesh_vertices, mesh_indices, image_height, image_width, eye, center, up, fov_y_degrees, vertex_colors,
                      face_colors, surface_color, light_direction, ambient, max_distance, bvh)


mesh_raycast = MeshRaycast.make_function("mesh_raycast")
