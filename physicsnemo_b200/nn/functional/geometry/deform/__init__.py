"""Point deformation, surface projection and deformation-energy functionals
(parity: ``physicsnemo/nn/functional/geometry/deform/__init__.py``)."""
from .energy import (ClosedSurfaceVolumeEnergy, SimplexInversionEnergy, SimplexMeasureEnergy, SimplexStrainEnergy,
                     SurfaceBendingEnergy, TotalMeasureEnergy, closed_surface_volume_energy, simplex_inversion_energy,
                     simplex_measure_energy, simplex_strain_energy, surface_bending_energy, total_measure_energy)
from .fields import (DisplacePoints, FreeFormDeformPoints, MorphPoints, RadialBasisFunctionDeformPoints, displace_points,
                     free_form_deform_points, morph_points, radial_basis_function_deform_points)
from .surface import ShrinkwrapPoints, SobolevDeformPoints, shrinkwrap_points, sobolev_deform_points

__all__ = [
    "ClosedSurfaceVolumeEnergy", "DisplacePoints", "FreeFormDeformPoints", "MorphPoints", "RadialBasisFunctionDeformPoints",
    "ShrinkwrapPoints", "SimplexInversionEnergy", "SimplexMeasureEnergy", "SimplexStrainEnergy", "SobolevDeformPoints",
    "SurfaceBendingEnergy", "TotalMeasureEnergy", "closed_surface_volume_energy", "displace_points",
    "free_form_deform_points", "morph_points", "radial_basis_function_deform_points", "shrinkwrap_points",
    "simplex_inversion_energy", "simplex_measure_energy", "simplex_strain_energy", "sobolev_deform_points",
    "surface_bending_energy", "total_measure_energy",
]
