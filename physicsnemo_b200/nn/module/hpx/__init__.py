from .layers import HEALPixLayer
from .padding import HEALPixFoldFaces, HEALPixPadding, HEALPixPaddingv2, HEALPixUnfoldFaces, padding_index_table
from .pool import HEALPixAvgPool, HEALPixMaxPool

__all__ = ["HEALPixLayer", "HEALPixFoldFaces", "HEALPixPadding", "HEALPixPaddingv2", "HEALPixUnfoldFaces", "HEALPixAvgPool",
           "HEALPixMaxPool", "padding_index_table"]
from .tokenizer import (CalendarEmbedding, FrequencyEmbedding, HEALPixPatchDetokenizer, HEALPixPatchTokenizer,  # noqa: E402
                        healpix_xy_lonlat)

__all__ += ["CalendarEmbedding", "FrequencyEmbedding", "HEALPixPatchDetokenizer", "HEALPixPatchTokenizer", "healpix_xy_lonlat"]
