"""Sequential composition of transforms (parity: ``physicsnemo/datapipes/transforms/compose.py``)."""
from __future__ import annotations

from typing import Any, Iterator, Sequence

import torch

from .._rng import fork_generator
from ..registry import register
from ..tensordict import TensorDict
from .base import Transform


@register()
class Compose(Transform):
    def __init__(self, transforms: Sequence[Transform]) -> None:
        super().__init__()
        for i, t in enumerate(transforms):
            if not isinstance(t, Transform):
                raise TypeError(f"All items must be Transform instances, got {type(t).__name__} at index {i}")
        self.transforms = list(transforms)

    def __call__(self, data: TensorDict) -> TensorDict:
        for t in self.transforms:
            data = t(data)
        return data

    @property
    def stochastic(self) -> bool:
        return any(t.stochastic for t in self.transforms)

    def set_generator(self, generator: torch.Generator) -> None:
        for child, t in zip(fork_generator(generator, len(self.transforms)), self.transforms):
            t.set_generator(child)

    def set_epoch(self, epoch: int) -> None:
        for t in self.transforms:
            t.set_epoch(epoch)

    def to(self, device) -> "Compose":
        super().to(device)
        for t in self.transforms:
            t.to(device)
        return self

    def __getitem__(self, index: int) -> Transform:
        return self.transforms[index]

    def __len__(self) -> int:
        return len(self.transforms)

    def __iter__(self) -> Iterator[Transform]:
        return iter(self.transforms)

    def append(self, transform: Transform) -> None:
        if not isinstance(transform, Transform):
            raise TypeError(f"Expected Transform, got {type(transform).__name__}")
        self.transforms.append(transform)

    def state_dict(self) -> dict[str, Any]:
        return {"transforms": [t.state_dict() for t in self.transforms]}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        for t, sd in zip(self.transforms, state_dict.get("transforms", [])):
            t.load_state_dict(sd)

    def extra_repr(self) -> str:
        return ", ".join(repr(t) for t in self.transforms)
