from .domino_datapipe import DoMINODataConfig, DoMINODataPipe, compute_scaling_factors
from .transolver_datapipe import TransolverDataConfig, TransolverDataPipe

__all__ = ["DoMINODataConfig", "DoMINODataPipe", "TransolverDataConfig", "TransolverDataPipe", "compute_scaling_factors"]
