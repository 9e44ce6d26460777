from .branches import SpatialBranch
from .deeponet import DeepONet
from .fno4d import FNO4DWrapper

__all__ = ["DeepONet", "SpatialBranch", "FNO4DWrapper"]
