from .diffusion_unets import DiffusionUNet3D
from .xdeeponet import DeepONet, FNO4DWrapper, SpatialBranch
from .healda import HealDA, VideoDiT, VideoHealDA
from .strata import Strata, StrataTransformer3D
from .tedm import tEDMPrecondSuperRes, tEDMResidualLoss

__all__ = ["HealDA", "VideoDiT", "VideoHealDA", "Strata", "StrataTransformer3D", "DeepONet", "FNO4DWrapper", "SpatialBranch", "DiffusionUNet3D", "tEDMPrecondSuperRes", "tEDMResidualLoss"]
