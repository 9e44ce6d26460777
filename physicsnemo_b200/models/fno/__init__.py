from .fno import FNO
