from .config import DEFAULT_MODEL_PARAMS, Config
from .model import (AggregationModel, DoMINO, GeoConvOut, GeometryRep, GeoProcessor, LocalGeometryEncoding, LocalPointConv,
                    MultiGeometryEncoding, SolutionCalculatorSurface, SolutionCalculatorVolume, scale_sdf)

__all__ = ["AggregationModel", "Config", "DEFAULT_MODEL_PARAMS", "DoMINO", "GeoConvOut", "GeoProcessor", "GeometryRep",
           "LocalGeometryEncoding", "LocalPointConv", "MultiGeometryEncoding", "SolutionCalculatorSurface",
           "SolutionCalculatorVolume", "scale_sdf"]
