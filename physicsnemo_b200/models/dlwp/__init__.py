from .dlwp import DLWP
