"""Several optimizers behind one ``Optimizer`` interface (e.g. Muon for matrices, Adam for the rest).

Parity: ``physicsnemo/optim/combined_optimizer.py:23-318`` — disjoint parameter sets are enforced,
``param_groups`` is the concatenation (so LR schedulers work), ``state_dict`` nests the members'
state under ``"optimizers"``, and groups cannot be added after construction.  The
``torch_compile_kwargs`` argument is accepted for signature parity and ignored: steps run eagerly.
"""
from typing import Any, Callable, Sequence

from torch.optim import Optimizer


class CombinedOptimizer(Optimizer):
    def __init__(self, optimizers: Sequence[Optimizer], torch_compile_kwargs: dict[str, Any] | None = None):
        if not optimizers:
            raise ValueError("`optimizers` must contain at least one optimizer.")
        owner: dict[int, int] = {}
        for oi, opt in enumerate(optimizers):
            for gi, group in enumerate(opt.param_groups):
                for p in group["params"]:
                    if id(p) in owner:
                        raise ValueError(
                            f"Parameter appears in multiple optimizers. Found duplicate in optimizer {oi}, group {gi}. "
                            "Each parameter must belong to exactly one optimizer to avoid being updated multiple times per step.")
                    owner[id(p)] = oi
        self.optimizers = optimizers
        self._torch_compile_kwargs = torch_compile_kwargs
        self._initializing = True
        try:
            super().__init__([g for opt in optimizers for g in opt.param_groups], defaults={})
        finally:
            self._initializing = False
        self.step_fns: list[Callable] = [opt.step for opt in optimizers]

    def zero_grad(self, set_to_none: bool = True) -> None:
        for opt in self.optimizers:
            opt.zero_grad(set_to_none=set_to_none)

    def step(self, closure: Callable[[], float] | None = None) -> float | None:
        loss = None
        for fn in self.step_fns:
            out = fn() if closure is None else fn(closure)
            if out is not None:
                loss = out
        return loss

    def add_param_group(self, param_group: dict[str, Any]) -> None:
        if getattr(self, "_initializing", False):
            return super().add_param_group(param_group)
        raise NotImplementedError(
            "CombinedOptimizer does not support add_param_group() after initialization, since it is ambiguous which "
            "optimizer should handle the new group.\nAdd parameters to the underlying optimizers before creating the "
            "CombinedOptimizer.")

    def state_dict(self) -> dict[str, Any]:
        return {"optimizers": [opt.state_dict() for opt in self.optimizers]}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        if "optimizers" not in state_dict:
            raise KeyError(f"Expected state_dict to contain 'optimizers' key, but got keys: {list(state_dict.keys())}")
        states = state_dict["optimizers"]
        if len(states) != len(self.optimizers):
            raise ValueError(f"State dict contains {len(states)} optimizer(s), but this CombinedOptimizer has "
                             f"{len(self.optimizers)} optimizer(s). Cannot load state from a different optimizer configuration.")
        for opt, sd in zip(self.optimizers, states):
            opt.load_state_dict(sd)
        self.param_groups = [g for opt in self.optimizers for g in opt.param_groups]

    def __repr__(self) -> str:
        return f"CombinedOptimizer({', '.join(type(o).__name__ for o in self.optimizers)})"
