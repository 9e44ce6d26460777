"""Observation filtering, featurisation and the two-stage (host, device) batch transform."""
from .obs_features import N_FEATURES, N_FEATURES_EXT, compute_unified_metadata, compute_unified_metadata_reference, local_solar_time

__all__ = ["N_FEATURES", "N_FEATURES_EXT", "compute_unified_metadata", "compute_unified_metadata_reference", "local_solar_time"]
