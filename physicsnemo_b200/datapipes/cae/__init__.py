from .cae_dataset import (BackendReader, CAEDataset, NpyDirectoryReader, NpyFileReader, NpzFileReader, ZarrFileReader,
                          compute_mean_std_min_max)
from .domino_datapipe import DoMINODataConfig, DoMINODataPipe, compute_scaling_factors
from .transolver_datapipe import TransolverDataConfig, TransolverDataPipe

__all__ = ["BackendReader", "CAEDataset", "DoMINODataConfig", "DoMINODataPipe", "NpyDirectoryReader", "NpyFileReader", "NpzFileReader",
           "TransolverDataConfig", "TransolverDataPipe", "ZarrFileReader", "compute_mean_std_min_max", "compute_scaling_factors"]
