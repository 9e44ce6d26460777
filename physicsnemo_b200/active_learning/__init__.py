"""Active learning: a driver cycling training, metrology, query and labelling phases."""
from ._registry import registry
from .config import DriverConfig, OptimizerConfig, StrategiesConfig, TrainingConfig
from .driver import Driver
from .loop import DefaultTrainingLoop

__all__ = ["registry", "Driver", "DefaultTrainingLoop", "DriverConfig", "OptimizerConfig", "StrategiesConfig",
           "TrainingConfig"]
