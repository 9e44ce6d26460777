from .base import Transform
from .compose import Compose
from .standard import (BoundingBoxFilter, BroadcastGlobalFeatures, CenterOfMass, ComputeNormals, ComputeSDF, ConcatFields,
                       ConstantField, CreateGrid, FieldSlice, KNearestNeighbors, Normalize, Purge, Rename, Scale,
                       SubsamplePoints, Translate, shuffle_array)

__all__ = ["Transform", "Compose", "Normalize", "SubsamplePoints", "ConcatFields", "FieldSlice", "BroadcastGlobalFeatures",
           "Rename", "Purge", "ConstantField", "Translate", "Scale", "BoundingBoxFilter", "CreateGrid", "KNearestNeighbors",
           "CenterOfMass", "ComputeSDF", "ComputeNormals", "shuffle_array"]
