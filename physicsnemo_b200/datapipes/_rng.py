"""Deterministic, coordinate-addressed random streams (parity: ``physicsnemo/datapipes/_rng.py``): the seed of any
(epoch, sample, transform) is a pure function of the base seed and its coordinates, so results do not depend on
worker scheduling."""
from __future__ import annotations

from typing import List, Union

import numpy as np
import torch


def derive_seed(base_seed: int, *coords: int) -> int:
    """64-bit seed hashed (NumPy ``SeedSequence``) from the base seed followed by the coordinates."""
    entropy = [int(base_seed)]
    entropy.extend(int(c) for c in coords)
    words = np.random.SeedSequence(entropy).generate_state(1, dtype=np.uint64)
    return int(words[0])


def spawn_generator(base_seed: int, *coords: int, device: Union[torch.device, str] = "cpu") -> torch.Generator:
    """A fresh generator on ``device`` seeded for the given coordinates."""
    return torch.Generator(device=device).manual_seed(derive_seed(base_seed, *coords))   # manual_seed returns the generator


def fork_generator(parent: torch.Generator, n: int) -> List[torch.Generator]:
    """``n`` independent children of ``parent``: child ``i`` is addressed by (``parent``'s initial seed, ``i``)."""
    root, where = parent.initial_seed(), parent.device
    children: List[torch.Generator] = []
    for child in range(n):
        children.append(spawn_generator(root, child, device=where))
    return children
