from .base import Reader
from .hdf5 import HDF5Reader
from .numpy import NumpyReader
from .vtk import DomainMeshReader, MeshReader, VTKReader
from .zarr import TensorStoreZarrReader, ZarrReader

__all__ = ["Reader", "HDF5Reader", "NumpyReader", "VTKReader", "MeshReader", "DomainMeshReader", "ZarrReader",
           "TensorStoreZarrReader"]
