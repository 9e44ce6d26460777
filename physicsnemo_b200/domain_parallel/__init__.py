"""Alias of ``physicsnemo_b200.parallel`` under the reference's package name."""
from ..parallel import *  # noqa: F401,F403
from ..parallel import __all__  # noqa: F401
