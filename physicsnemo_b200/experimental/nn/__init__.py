from .rope import (apply_rope, build_axial_rope_cos_sin_2d_continuous, build_rope_cos_sin_1d_continuous, spherical_centroid,
                   stereographic_projection)

from .diffusion_unet_3d_blocks import Conv3D, GroupNorm3D, UNetAttention3D, UNetBlock3D

__all__ = ["Conv3D", "GroupNorm3D", "UNetAttention3D", "UNetBlock3D", "apply_rope", "build_axial_rope_cos_sin_2d_continuous", "build_rope_cos_sin_1d_continuous", "spherical_centroid",
           "stereographic_projection"]
