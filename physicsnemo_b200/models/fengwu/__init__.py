from .fengwu import Fengwu
