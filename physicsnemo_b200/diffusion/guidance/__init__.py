from .dps_guidance import DataConsistencyDPSGuidance, DPSGuidance, DPSScorePredictor, ModelConsistencyDPSGuidance

__all__ = ["DPSGuidance", "DPSScorePredictor", "ModelConsistencyDPSGuidance", "DataConsistencyDPSGuidance"]
