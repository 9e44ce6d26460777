"""SO(2) / SO(3) equivariant layers on spherical-harmonic grids (``[B, l, m, (real, imag), channel]``)."""

from .activation import GateActivation
from .grid import make_grid_mask
from .layer_norm import (EquivariantLayerNorm, EquivariantLayerNormTied, EquivariantRMSNorm, FusedEquivariantLayerNorm,
                         FusedEquivariantLayerNormTied, FusedEquivariantRMSNorm, make_degree_balance_weight, make_m0_imag_mask)
from .so2_conv import SO2Convolution
from .so3_block import SO3ConvolutionBlock
from .so3_linear import SO3LinearGrid
from .wigner import EdgeRotation, compute_wigner_d_matrices, edge_vectors_to_euler_angles, rotate_grid_coefficients

__all__ = ["EdgeRotation", "EquivariantLayerNorm", "EquivariantLayerNormTied", "EquivariantRMSNorm", "FusedEquivariantLayerNorm",
           "FusedEquivariantLayerNormTied", "FusedEquivariantRMSNorm", "GateActivation", "SO2Convolution", "SO3ConvolutionBlock",
           "SO3LinearGrid", "compute_wigner_d_matrices", "edge_vectors_to_euler_angles", "make_degree_balance_weight",
           "make_grid_mask", "make_m0_imag_mask", "rotate_grid_coefficients"]
