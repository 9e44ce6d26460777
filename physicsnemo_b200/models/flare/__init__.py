from .flare import FLARE
