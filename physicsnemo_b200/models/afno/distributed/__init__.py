from .afno import DistributedAFNO  # noqa: F401
