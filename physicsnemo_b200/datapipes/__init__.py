"""GPU-centric data loading: Readers → Transforms → Dataset → DataLoader, plus on-device PDE data generators."""
from .collate import (Collator, ConcatCollator, DefaultCollator, FunctionCollator, concat_collate, default_collate,
                      get_collator)
from .dataloader import DataLoader
from .dataset import Dataset
from .multi_dataset import MultiDataset
from .protocols import DatasetBase, IterableDatasetBase
from .readers import (DomainMeshReader, HDF5Reader, MeshReader, NumpyReader, Reader, TensorStoreZarrReader, VTKReader,
                      ZarrReader)
from .registry import COMPONENT_REGISTRY, ComponentRegistry, register, register_resolvers
from .tensordict import TensorDict
from .transforms import *  # noqa: F401,F403
from .transforms import __all__ as _transform_names

register_resolvers()

__all__ = ["TensorDict", "DatasetBase", "IterableDatasetBase", "Dataset", "DataLoader", "MultiDataset", "Reader",
           "NumpyReader", "HDF5Reader", "ZarrReader", "TensorStoreZarrReader", "VTKReader", "MeshReader", "DomainMeshReader",
           "Collator", "DefaultCollator", "ConcatCollator", "FunctionCollator", "default_collate", "concat_collate",
           "get_collator", "COMPONENT_REGISTRY", "ComponentRegistry", "register", "register_resolvers", *_transform_names]
