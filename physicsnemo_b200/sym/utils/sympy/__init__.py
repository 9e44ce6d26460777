from .torch_printer import SympyToTorch, torch_lambdify  # noqa: F401
