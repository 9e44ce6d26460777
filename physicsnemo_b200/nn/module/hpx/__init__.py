from .layers import HEALPixLayer
from .padding import HEALPixFoldFaces, HEALPixPadding, HEALPixPaddingv2, HEALPixUnfoldFaces, padding_index_table
from .pool import HEALPixAvgPool, HEALPixMaxPool

__all__ = ["HEALPixLayer", "HEALPixFoldFaces", "HEALPixPadding", "HEALPixPaddingv2", "HEALPixUnfoldFaces", "HEALPixAvgPool",
           "HEALPixMaxPool", "padding_index_table"]
