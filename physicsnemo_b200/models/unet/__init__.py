from .unet import UNet
