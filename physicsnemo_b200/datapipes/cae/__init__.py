from .domino_datapipe import DoMINODataConfig, DoMINODataPipe, compute_scaling_factors

__all__ = ["DoMINODataConfig", "DoMINODataPipe", "compute_scaling_factors"]
