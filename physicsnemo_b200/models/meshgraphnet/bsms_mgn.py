"""Import location kept for parity with ``physicsnemo/models/meshgraphnet/bsms_mgn.py``."""
from .variants import *  # noqa: F401,F403
from .variants import BiStrideMeshGraphNet, HybridMeshGraphNet, HybridMeshGraphNetProcessor, MeshGraphKAN  # noqa: F401
