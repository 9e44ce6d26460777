"""Deterministic, coordinate-addressed random streams (parity: ``physicsnemo/datapipes/_rng.py``): the seed of any
(epoch, sample, transform) is a pure function of the base seed and its coordinates, so results do not depend on
worker scheduling."""
from __future__ import annotations

import numpy as np
import torch


def derive_seed(base_seed: int, *coords: int) -> int:
    seq = np.random.SeedSequence([int(base_seed), *(int(c) for c in coords)])
    return int(seq.generate_state(1, dtype=np.uint64)[0])


def spawn_generator(base_seed: int, *coords: int, device: torch.device | str = "cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(derive_seed(base_seed, *coords))
    return g


def fork_generator(parent: torch.Generator, n: int) -> list[torch.Generator]:
    base = parent.initial_seed()
    return [spawn_generator(base, i, device=parent.device) for i in range(n)]
