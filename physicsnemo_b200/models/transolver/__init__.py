from .transolver import Transolver, TransolverBlock

__all__ = ["Transolver", "TransolverBlock"]
