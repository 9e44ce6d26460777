"""Import location kept for parity with ``physicsnemo/models/dpot/dpot3d.py``."""
from .dpot import AFNO3DLayer, Block3D, ConvMlp3D, DPOT3DMeta, DPOTNet3D, PatchEmbed3D, TimeAggregator  # noqa: F401
