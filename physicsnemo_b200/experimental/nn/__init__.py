from .rope import (apply_rope, build_axial_rope_cos_sin_2d_continuous, build_rope_cos_sin_1d_continuous, spherical_centroid,
                   stereographic_projection)

__all__ = ["apply_rope", "build_axial_rope_cos_sin_2d_continuous", "build_rope_cos_sin_1d_continuous", "spherical_centroid",
           "stereographic_projection"]
