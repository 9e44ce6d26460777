from .gmm import TorchGMM
from .ood_guard import OODGuard, OODGuardConfig

__all__ = ["OODGuard", "OODGuardConfig", "TorchGMM"]
