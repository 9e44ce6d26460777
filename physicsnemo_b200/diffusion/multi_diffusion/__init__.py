from .dps_guidance import (MultiDiffusionDataConsistencyDPSGuidance, MultiDiffusionDPSGuidance,
                           MultiDiffusionDPSScorePredictor, MultiDiffusionModelConsistencyDPSGuidance)
from .losses import MultiDiffusionMSEDSMLoss, MultiDiffusionWeightedMSEDSMLoss
from .models import ConditionDict, MultiDiffusionModel2D
from .patching import BasePatching2D, GridPatching2D, RandomPatching2D, image_batching, image_fuse
from .predictor import MultiDiffusionPredictor

__all__ = ["BasePatching2D", "ConditionDict", "GridPatching2D", "MultiDiffusionDPSGuidance", "MultiDiffusionDPSScorePredictor",
           "MultiDiffusionDataConsistencyDPSGuidance", "MultiDiffusionModelConsistencyDPSGuidance", "MultiDiffusionMSEDSMLoss", "MultiDiffusionModel2D",
           "MultiDiffusionPredictor", "MultiDiffusionWeightedMSEDSMLoss", "RandomPatching2D", "image_batching", "image_fuse"]
