from .darcy import Darcy2D
from .kelvin_helmholtz import KelvinHelmholtz2D
