from .dit import DiT
