from .variational_gp_head import GPDistribution, GPPrediction, VariationalGPHead

__all__ = ["GPDistribution", "GPPrediction", "VariationalGPHead"]
