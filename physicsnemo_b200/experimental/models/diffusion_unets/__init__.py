from .diffusion_unet_3d import DiffusionUNet3D

__all__ = ["DiffusionUNet3D"]
