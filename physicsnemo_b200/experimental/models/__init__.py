from .diffusion_unets import DiffusionUNet3D
from .xdeeponet import DeepONet, FNO4DWrapper, SpatialBranch
from .healda import HealDA, VideoDiT, VideoHealDA
from .strata import Strata, StrataTransformer3D
from .aerojepa import AeroJEPA, AeroJEPATrunk
from .globe import GLOBE
from .tedm import tEDMPrecondSuperRes, tEDMResidualLoss

__all__ = ["AeroJEPA", "AeroJEPATrunk", "GLOBE", "HealDA", "VideoDiT", "VideoHealDA", "Strata", "StrataTransformer3D", "DeepONet", "FNO4DWrapper", "SpatialBranch", "DiffusionUNet3D", "tEDMPrecondSuperRes", "tEDMResidualLoss"]
