from .topodiff import TopoDiff, UNetEncoder
