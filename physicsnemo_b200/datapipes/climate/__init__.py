from .era5 import ERA5Datapipe
from .synthetic import SyntheticWeatherDataLoader, SyntheticWeatherDataset

ERA5HDF5Datapipe = ERA5Datapipe

__all__ = ["ERA5Datapipe", "ERA5HDF5Datapipe", "SyntheticWeatherDataLoader", "SyntheticWeatherDataset"]
