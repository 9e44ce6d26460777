from .field_variational_gp_head import FieldVariationalGPHead, FieldVariationalGPPrediction
from .variational_gp_head import GPDistribution, GPPrediction, VariationalGPHead

__all__ = ["FieldVariationalGPHead", "FieldVariationalGPPrediction", "GPDistribution", "GPPrediction", "VariationalGPHead"]
