from .transforms import (CenterMesh, ComputeCellCentroids, ComputeSurfaceNormals, DropMeshFields, MeshToTensorDict, MeshTransform,
                         NormalizeMeshFields, RandomRotateMesh, RandomScaleMesh, RandomTranslateMesh, RenameMeshFields, RestructureTensorDict,
                         RotateMesh, ScaleMesh, SetGlobalField, SubsampleMesh, TranslateMesh)

__all__ = ["CenterMesh", "ComputeCellCentroids", "ComputeSurfaceNormals", "DropMeshFields", "MeshToTensorDict", "MeshTransform",
           "NormalizeMeshFields", "RandomRotateMesh", "RandomScaleMesh", "RandomTranslateMesh", "RenameMeshFields", "RestructureTensorDict",
           "RotateMesh", "ScaleMesh", "SetGlobalField", "SubsampleMesh", "TranslateMesh"]
