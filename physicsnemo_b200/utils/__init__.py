from .capture import StaticCaptureEvaluateNoGrad, StaticCaptureTraining
from .checkpoint import get_checkpoint_dir, load_checkpoint, load_model_weights, save_checkpoint
from .logging import LaunchLogger, PythonLogger, RankZeroLoggingWrapper
from .profiling import Profiler

__all__ = [
    "StaticCaptureTraining", "StaticCaptureEvaluateNoGrad", "get_checkpoint_dir", "load_checkpoint",
    "load_model_weights", "save_checkpoint", "LaunchLogger", "PythonLogger", "RankZeroLoggingWrapper", "Profiler",
]
