"""HealDA data pipeline: observation + state loading, two-stage transforms, restartable sampling, prefetching.

Parity: ``physicsnemo/experimental/datapipes/healda/__init__.py``.
"""
from .configs import QCLimits, SensorConfig, SensorRegistry, VARIABLE_CONFIGS
from .dataset import ObsERA5Dataset, identity_collate
from .loaders import ArrayStateStore, TableObsLoader
from .prefetch import prefetch_map
from .protocols import DeviceTransform, ObsLoader, Transform
from .samplers import RestartableDistributedSampler
from .transforms.era5_obs import ERA5ObsTransform
from .types import Batch, BatchInfo, TimeUnit, UnifiedObservation, VariableConfig, empty_batch, split_by_sensor

__all__ = ["ObsERA5Dataset", "identity_collate", "ArrayStateStore", "TableObsLoader", "ERA5ObsTransform", "prefetch_map",
           "ObsLoader", "Transform", "DeviceTransform", "RestartableDistributedSampler", "Batch", "BatchInfo", "TimeUnit",
           "UnifiedObservation", "VariableConfig", "empty_batch", "split_by_sensor", "SensorConfig", "SensorRegistry", "QCLimits",
           "VARIABLE_CONFIGS"]
