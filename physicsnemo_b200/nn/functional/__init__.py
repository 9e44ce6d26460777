"""Functional operator surface (parity: ``physicsnemo/nn/functional/__init__.py``): every functional of the
sub-packages under one namespace."""
from .derivatives import (mesh_green_gauss_gradient, mesh_lsq_gradient, meshless_fd_derivatives, rectilinear_grid_curl,
                          rectilinear_grid_divergence, rectilinear_grid_gradient, rectilinear_grid_laplacian,
                          spectral_grid_gradient, uniform_grid_curl, uniform_grid_divergence, uniform_grid_gradient,
                          uniform_grid_laplacian)
from .equivariant_ops import legendre_polynomials, polar_and_dipole_basis, smooth_log, spherical_basis, vector_project
from .fourier_spectral import imag, irfft, irfft2, real, rfft, rfft2, view_as_complex
from .geometry import (closed_surface_volume_energy, displace_points, farthest_point_sampling, free_form_deform_points,
                       mesh_poisson_disk_sample, mesh_to_voxel_fraction, morph_points,
                       radial_basis_function_deform_points, ray_mesh_intersect, remeshing, shrinkwrap_points,
                       signed_distance_field, simplex_inversion_energy, simplex_measure_energy, simplex_strain_energy,
                       sobolev_deform_points, surface_bending_energy, total_measure_energy)
from .interpolation import grid_to_point_interpolation, interpolation, point_to_grid_interpolation
from .natten import na1d, na2d, na3d
from .neighbors import knn, radius_search
from .regularization_parameterization import drop_path, weight_fact
from .rendering import (isosurface_render, line_integral_convolution, mesh_raycast, point_cloud_render,
                        scalar_field_to_rgba, vector_field_to_rgba, volume_render, wireframe_render)
from .weighted_multinomial import WeightedMultinomial, weighted_multinomial

__all__ = [
    "WeightedMultinomial", "closed_surface_volume_energy", "displace_points", "drop_path", "farthest_point_sampling",
    "free_form_deform_points", "grid_to_point_interpolation", "imag", "interpolation", "irfft", "irfft2",
    "isosurface_render", "knn", "legendre_polynomials", "line_integral_convolution", "mesh_green_gauss_gradient",
    "mesh_lsq_gradient", "mesh_poisson_disk_sample", "mesh_raycast", "mesh_to_voxel_fraction", "meshless_fd_derivatives",
    "morph_points", "na1d", "na2d", "na3d", "point_cloud_render", "point_to_grid_interpolation", "polar_and_dipole_basis",
    "radial_basis_function_deform_points", "radius_search", "ray_mesh_intersect", "real", "rectilinear_grid_curl",
    "rectilinear_grid_divergence", "rectilinear_grid_gradient", "rectilinear_grid_laplacian", "remeshing", "rfft", "rfft2",
    "scalar_field_to_rgba", "shrinkwrap_points", "signed_distance_field", "simplex_inversion_energy",
    "simplex_measure_energy", "simplex_strain_energy", "smooth_log", "sobolev_deform_points", "spectral_grid_gradient",
    "spherical_basis", "surface_bending_energy", "total_measure_energy", "uniform_grid_curl", "uniform_grid_divergence",
    "uniform_grid_gradient", "uniform_grid_laplacian", "vector_field_to_rgba", "vector_project", "view_as_complex",
    "volume_render", "weight_fact", "weighted_multinomial", "wireframe_render",
]
