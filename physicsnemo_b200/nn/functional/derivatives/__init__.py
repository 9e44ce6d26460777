"""Derivative functionals on grids, point stencils and meshes."""
from .mesh_gradients import MeshGreenGaussGradient, MeshLSQGradient, mesh_green_gauss_gradient, mesh_lsq_gradient
from .meshless_spectral import (MeshlessFDDerivatives, SpectralGridGradient, meshless_fd_derivatives,
                                meshless_fd_stencil_points, spectral_grid_gradient)
from .rectilinear_grid import (RectilinearGridCurl, RectilinearGridDivergence, RectilinearGridGradient,
                               RectilinearGridLaplacian, rectilinear_grid_curl, rectilinear_grid_divergence,
                               rectilinear_grid_gradient, rectilinear_grid_laplacian)
from .uniform_grid import (UniformGridCurl, UniformGridDivergence, UniformGridGradient, UniformGridLaplacian,
                           uniform_grid_curl, uniform_grid_divergence, uniform_grid_gradient, uniform_grid_laplacian)
