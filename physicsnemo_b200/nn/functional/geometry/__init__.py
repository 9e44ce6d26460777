from .farthest_point_sampling import FarthestPointSampling, farthest_point_sampling
from .sdf import RayMeshIntersect, SignedDistanceField, ray_mesh_intersect, signed_distance_field
from .deform import *  # noqa: F401,F403
from .deform import __all__ as _deform_all
