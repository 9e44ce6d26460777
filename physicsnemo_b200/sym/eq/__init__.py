from .gradients import GradientCalculator, compute_connectivity_tensor  # noqa: F401
from .pde import PDE  # noqa: F401
from .phy_informer import PhysicsInformer  # noqa: F401
