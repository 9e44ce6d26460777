"""Sequential composition of transforms (parity: ``physicsnemo/datapipes/transforms/compose.py``)."""
from __future__ import annotations

from typing import Any, Iterator, Sequence

import torch

from .._rng import fork_generator
from ..registry import register
from ..tensordict import TensorDict
from .base import Transform


def _require_transform(obj, where: str = "") -> None:
    if not isinstance(obj, Transform):
        raise TypeError(f"Expected Transform, got {type(obj).__name__}" if not where
                        else f"All items must be Transform instances, got {type(obj).__name__} at index {where}")


@register()
class Compose(Transform):
    """Apply the member transforms in order; a list-like container of them."""

    def __init__(self, transforms: Sequence[Transform]) -> None:
        super().__init__()
        self.transforms = []
        for position, member in enumerate(transforms):
            _require_transform(member, str(position))
            self.transforms.append(member)

    def __call__(self, data: TensorDict) -> TensorDict:
        out = data
        for member in self.transforms:
            out = member(out)
        return out

    # container protocol
    def __len__(self) -> int:
        return len(self.transforms)

    def __iter__(self) -> Iterator[Transform]:
        yield from self.transforms

    def __getitem__(self, index: int) -> Transform:
        return self.transforms[index]

    def append(self, transform: Transform) -> None:
        _require_transform(transform)
        self.transforms.append(transform)

    # everything else fans out to the members
    @property
    def stochastic(self) -> bool:
        return any(member.stochastic for member in self.transforms)

    def set_generator(self, generator: torch.Generator) -> None:
        """Every member gets its own stream forked from ``generator``, so adding a member does not shift the others' draws."""
        streams = fork_generator(generator, len(self.transforms))
        for member, stream in zip(self.transforms, streams):
            member.set_generator(stream)

    def set_epoch(self, epoch: int) -> None:
        for member in self.transforms:
            member.set_epoch(epoch)

    def to(self, device) -> "Compose":
        super().to(device)
        for member in self.transforms:
            member.to(device)
        return self

    def state_dict(self) -> dict[str, Any]:
        return {"transforms": [member.state_dict() for member in self.transforms]}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        for member, saved in zip(self.transforms, state_dict.get("transforms", ())):
            member.load_state_dict(saved)

    def extra_repr(self) -> str:
        return ", ".join(map(repr, self.transforms))
