from .console import PythonLogger, RankZeroLoggingWrapper
from .launch import LaunchLogger

__all__ = ["PythonLogger", "RankZeroLoggingWrapper", "LaunchLogger"]
