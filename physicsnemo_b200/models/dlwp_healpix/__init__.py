from .healpix_unet import HEALPixRecUNet, HEALPixUNet
from . import layers

__all__ = ["HEALPixRecUNet", "HEALPixUNet", "layers"]
