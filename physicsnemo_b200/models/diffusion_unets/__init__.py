from .dhariwal_unet import DhariwalUNet
from .song_unet import SongUNet, SongUNetPosEmbd, SongUNetPosLtEmbd
from .unet import CorrDiffRegressionUNet, StormCastUNet, UNet

__all__ = ["SongUNet", "SongUNetPosEmbd", "SongUNetPosLtEmbd", "DhariwalUNet", "CorrDiffRegressionUNet", "UNet",
           "StormCastUNet"]
