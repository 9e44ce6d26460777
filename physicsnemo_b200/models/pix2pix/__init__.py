from .pix2pix import Pix2Pix
from .pix2pixunet import Pix2PixUnet
