from .mesh_reduced import Mesh_Reduced  # noqa: F401
from .temporal_model import Sequence_Model  # noqa: F401
