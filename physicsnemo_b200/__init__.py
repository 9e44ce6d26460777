"""physicsnemo_b200: a Blackwell (sm_100a) native physics-ML framework.

Public surface follows NVIDIA PhysicsNeMo (``physicsnemo/__init__.py``):
``Module``, ``ModelMetaData`` and the sub-packages ``core``, ``distributed``,
``domain_parallel`` (alias of ``parallel``), ``nn``, ``models``, ``diffusion``,
``utils``, ``metrics``, ``optim``, ``datapipes``, ``mesh``, ``sym``.  Importing
the package needs only ``torch`` and ``numpy``.
"""
import os as _os

from .core.meta import ModelMetaData
from .core.module import Module

__version__ = "2.2.0a0"

if _os.getenv("PHYSICSNEMO_ENABLE_COMPAT") in {"1", "true", "True", "YES", "yes", "on", "ON"}:
    from .compat import install as _compat_install

    _compat_install()

__all__ = ["Module", "ModelMetaData", "__version__"]
