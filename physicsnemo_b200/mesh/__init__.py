"""Simplicial meshes with tensor data: geometry, topology, calculus, generation, spatial queries, IO."""
from . import io, operations, primitives, spatial
from .domain_mesh import DomainMesh
from .fields import RankSpecDict, flatten_rank_spec, rank_counts, ranks_from_tensordict, validate_data_contains_ranks
from .mesh import MESH_FIELD_ASSOCIATIONS, Adjacency, Mesh, MeshFieldAssociation

__all__ = ["Mesh", "DomainMesh", "Adjacency", "MeshFieldAssociation", "MESH_FIELD_ASSOCIATIONS", "RankSpecDict",
           "flatten_rank_spec", "rank_counts", "ranks_from_tensordict", "validate_data_contains_ranks", "primitives",
           "operations", "spatial", "io"]
from . import generate, repair, tessellation  # noqa: E402,F401
from .generate import marching_cubes  # noqa: E402,F401
from . import calculus, subdivision  # noqa: E402,F401
from .subdivision import subdivide_linear, subdivide_loop  # noqa: E402,F401
from . import boundaries, cluster_tree, projections  # noqa: E402,F401
from .projections import embed, extrude, project  # noqa: E402,F401
from . import geometry, sampling  # noqa: E402,F401
