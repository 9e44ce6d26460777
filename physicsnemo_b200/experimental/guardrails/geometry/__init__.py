"""Geometry out-of-distribution guardrail on global shape descriptors of surface meshes."""

from .density_model import GeometryDensityModel
from .density_pce import TorchPCEDensityModel
from .feature_extraction import FEATURE_NAMES, FEATURE_VERSION, FeatureSchema, extract_features, feature_hash, validate_mesh
from .ood_detector import GeometryGuardrail

__all__ = ["FEATURE_NAMES", "FEATURE_VERSION", "FeatureSchema", "GeometryDensityModel", "GeometryGuardrail", "TorchPCEDensityModel",
           "extract_features", "feature_hash", "validate_mesh"]
