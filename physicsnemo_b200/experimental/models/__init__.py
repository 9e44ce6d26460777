from .diffusion_unets import DiffusionUNet3D
from .tedm import tEDMPrecondSuperRes, tEDMResidualLoss

__all__ = ["DiffusionUNet3D", "tEDMPrecondSuperRes", "tEDMResidualLoss"]
