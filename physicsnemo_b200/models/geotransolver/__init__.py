"""GeoTransolver: geometry-aware physics-attention transformer."""
from ...nn.module.gale import GALE, GALE_FA, GALEBlock, GALEStructuredMesh2D, GALEStructuredMesh3D
from .context_projector import (ContextProjector, GeometricFeatureProcessor, GlobalContextBuilder, MultiScaleFeatureExtractor,
                                StructuredContextProjector)
from .geotransolver import GeoTransolver, GeoTransolverMetaData

__all__ = ["GeoTransolver", "GeoTransolverMetaData", "GALE", "GALE_FA", "GALEBlock", "GALEStructuredMesh2D",
           "GALEStructuredMesh3D", "ContextProjector", "StructuredContextProjector", "GeometricFeatureProcessor",
           "MultiScaleFeatureExtractor", "GlobalContextBuilder"]
