"""Headless rendering functionals: every function returns plain image tensors."""
from .field_maps import (LineIntegralConvolution, ScalarFieldToRGBA, VectorFieldToRGBA, line_integral_convolution,
                         scalar_field_to_rgba, vector_field_to_rgba)
from .mesh_raycast import MeshRaycast, mesh_raycast
from .raster import PointCloudRender, WireframeRender, point_cloud_render, wireframe_render
from .raymarch import IsosurfaceRender, VolumeRender, isosurface_render, volume_render

__all__ = ["IsosurfaceRender", "LineIntegralConvolution", "MeshRaycast", "PointCloudRender", "ScalarFieldToRGBA",
           "VectorFieldToRGBA", "VolumeRender", "WireframeRender", "isosurface_render", "line_integral_convolution",
           "mesh_raycast", "point_cloud_render", "scalar_field_to_rgba", "vector_field_to_rgba", "volume_render",
           "wireframe_render"]
