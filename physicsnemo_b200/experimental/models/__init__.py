from .diffusion_unets import DiffusionUNet3D
from .xdeeponet import DeepONet, FNO4DWrapper, SpatialBranch
from .tedm import tEDMPrecondSuperRes, tEDMResidualLoss

__all__ = ["DeepONet", "FNO4DWrapper", "SpatialBranch", "DiffusionUNet3D", "tEDMPrecondSuperRes", "tEDMResidualLoss"]
