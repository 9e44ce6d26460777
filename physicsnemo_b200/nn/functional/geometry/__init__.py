"""Geometry functionals (parity: ``physicsnemo/nn/functional/geometry/__init__.py``)."""
from .deform import *  # noqa: F401,F403
from .deform import __all__ as _deform_all
from .farthest_point_sampling import FarthestPointSampling, farthest_point_sampling
from .mesh_poisson_disk_sample import MeshPoissonDiskSample, mesh_poisson_disk_sample
from .mesh_to_voxel_fraction import MeshToVoxelFraction, mesh_to_voxel_fraction
from .remeshing import Remeshing, remeshing
from .sdf import RayMeshIntersect, SignedDistanceField, ray_mesh_intersect, signed_distance_field

__all__ = [*_deform_all, "FarthestPointSampling", "MeshPoissonDiskSample", "MeshToVoxelFraction", "RayMeshIntersect",
           "Remeshing", "SignedDistanceField", "farthest_point_sampling", "mesh_poisson_disk_sample",
           "mesh_to_voxel_fraction", "ray_mesh_intersect", "remeshing", "signed_distance_field"]
