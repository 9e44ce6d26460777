from .meshgraphnet import MeshGraphNet, MeshGraphNetProcessor
from .variants import (BiStrideMeshGraphNet, HybridMeshGraphNet, HybridMeshGraphNetProcessor, MeshGraphKAN)

__all__ = ["MeshGraphNet", "MeshGraphNetProcessor", "BiStrideMeshGraphNet", "HybridMeshGraphNet",
           "HybridMeshGraphNetProcessor", "MeshGraphKAN"]
