from .afno import AFNO
from .distributed import DistributedAFNO
from .modafno import ModAFNO
from .modembed import ModEmbedNet

__all__ = ["AFNO", "DistributedAFNO", "ModAFNO", "ModEmbedNet"]
