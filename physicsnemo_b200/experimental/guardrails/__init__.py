from .geometry import GeometryDensityModel, GeometryGuardrail, TorchPCEDensityModel, extract_features
from .geotransolver_guard import GuardedGeoTransolver, attach_ood_guard
from .gmm import TorchGMM
from .ood_guard import OODGuard, OODGuardConfig

__all__ = ["GeometryDensityModel", "GeometryGuardrail", "TorchPCEDensityModel", "extract_features", "GuardedGeoTransolver", "OODGuard", "OODGuardConfig", "TorchGMM", "attach_ood_guard"]
