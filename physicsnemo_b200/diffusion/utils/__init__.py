from .model_wrappers import ConcatConditionWrapper
from .utils import InfiniteSampler, StackedRandomGenerator, apply_loss_weight

__all__ = ["ConcatConditionWrapper", "InfiniteSampler", "StackedRandomGenerator", "apply_loss_weight"]
