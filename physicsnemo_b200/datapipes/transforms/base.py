"""``Transform``: a callable ``TensorDict → TensorDict`` that can live on a device and own a random stream
(parity: ``physicsnemo/datapipes/transforms/base.py``)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Optional

import torch

from .._rng import derive_seed
from ..tensordict import TensorDict


def _relocate(value, device: torch.device):
    """Copy of an attribute on ``device`` when it is device-bound (tensor, dict of tensors, generator); else ``None``."""
    if isinstance(value, torch.Tensor):
        return value.to(device)
    if isinstance(value, torch.Generator):
        return torch.Generator(device=device).manual_seed(value.initial_seed())
    if isinstance(value, dict) and value and all(isinstance(v, torch.Tensor) for v in value.values()):
        return {k: v.to(device) for k, v in value.items()}
    return None


class Transform(ABC):
    """Base of all sample transforms.  A subclass that draws random numbers keeps its ``torch.Generator`` in
    ``self._generator`` (``None`` until the pipeline seeds it); that attribute is what marks it as stochastic."""

    def __init__(self) -> None:
        self._device: Optional[torch.device] = None

    @abstractmethod
    def __call__(self, data: TensorDict) -> TensorDict:
        raise NotImplementedError

    # -------------------------------------------------------------- randomness
    @property
    def stochastic(self) -> bool:
        return "_generator" in self.__dict__ or hasattr(type(self), "_generator")

    def set_generator(self, generator: torch.Generator) -> None:
        """Adopt the pipeline's generator (no-op for deterministic transforms); its seed anchors the per-epoch reseeding."""
        if not self.stochastic:
            return
        self._generator, self._seed_base = generator, generator.initial_seed()

    def set_epoch(self, epoch: int) -> None:
        """Reseed from ``(base seed, epoch)`` so that an epoch's draws do not depend on how earlier epochs ran."""
        gen = getattr(self, "_generator", None)
        if gen is None:
            return
        base = getattr(self, "_seed_base", None)
        if base is None:
            base = self._seed_base = gen.initial_seed()
        gen.manual_seed(derive_seed(base, epoch))

    # ------------------------------------------------------------------ device
    def to(self, device: torch.device | str) -> "Transform":
        self._device = torch.device(device)
        for name in list(vars(self)):
            moved = _relocate(getattr(self, name), self._device)
            if moved is not None:
                setattr(self, name, moved)
        return self

    @property
    def device(self) -> torch.device | None:
        return self._device

    # ------------------------------------------------------------------- state
    def state_dict(self) -> dict[str, Any]:
        return {}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        return None

    def extra_repr(self) -> str:
        return ""

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.extra_repr()})"
