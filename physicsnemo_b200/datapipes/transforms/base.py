"""``Transform``: a callable ``TensorDict → TensorDict`` that can live on a device and own a random stream
(parity: ``physicsnemo/datapipes/transforms/base.py``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Optional

import torch

from .._rng import derive_seed
from ..tensordict import TensorDict


class Transform(ABC):
    def __init__(self) -> None:
        self._device: Optional[torch.device] = None

    @abstractmethod
    def __call__(self, data: TensorDict) -> TensorDict:
        raise NotImplementedError

    @property
    def stochastic(self) -> bool:
        """Stochastic transforms declare a ``_generator`` attribute (possibly ``None`` until seeded)."""
        return hasattr(self, "_generator")

    def set_generator(self, generator: torch.Generator) -> None:
        if self.stochastic:
            self._generator = generator
            self._seed_base = generator.initial_seed()

    def set_epoch(self, epoch: int) -> None:
        if self.stochastic and self._generator is not None:
            if getattr(self, "_seed_base", None) is None:
                self._seed_base = self._generator.initial_seed()
            self._generator.manual_seed(derive_seed(self._seed_base, epoch))

    def to(self, device: torch.device | str) -> "Transform":
        self._device = torch.device(device)
        for name, value in list(self.__dict__.items()):
            if isinstance(value, torch.Tensor):
                setattr(self, name, value.to(self._device))
            elif isinstance(value, torch.Generator):
                g = torch.Generator(device=self._device)
                g.manual_seed(value.initial_seed())
                setattr(self, name, g)
            elif isinstance(value, dict) and value and all(isinstance(v, torch.Tensor) for v in value.values()):
                setattr(self, name, {k: v.to(self._device) for k, v in value.items()})
        return self

    @property
    def device(self) -> torch.device | None:
        return self._device

    def extra_repr(self) -> str:
        return ""

    def state_dict(self) -> dict[str, Any]:
        return {}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        return None

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}({self.extra_repr()})"
