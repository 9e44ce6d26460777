from .figconvunet import FIGConvUNet, GridFeaturesMemoryFormat

__all__ = ["FIGConvUNet", "GridFeaturesMemoryFormat"]
