"""GLOBE model and its kernels (parity: ``physicsnemo/experimental/models/globe/__init__.py``)."""
from .field_kernel import BarnesHutKernel, Kernel, MultiscaleKernel
from .model import GLOBE

__all__ = ["GLOBE", "Kernel", "BarnesHutKernel", "MultiscaleKernel"]
