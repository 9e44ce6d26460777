"""Index helpers shared by readers and sub-sampling transforms (parity: ``physicsnemo/datapipes/_indexing.py``)."""
from __future__ import annotations

import torch


def _cyclic_block_indices(total: int, k: int, start: int | None = None, device=None, *,
                          generator: torch.Generator | None = None) -> torch.Tensor:
    """``k`` consecutive indices of ``[0, total)`` starting at a uniformly random (or given) position and wrapping at
    the end: every element is included with probability exactly ``k / total`` while the selection stays one or two
    contiguous runs (friendly to memory-mapped and chunked stores)."""
    if total < 0 or k < 0:
        raise ValueError(f"total and k must be non-negative, got {total=} and {k=}.")
    if k > total:
        raise ValueError(f"Range size {total} is less than the requested block size {k}.")
    if start is not None and generator is not None:
        raise ValueError("start and generator are mutually exclusive.")
    if start is not None and not 0 <= start < total:
        raise ValueError(f"start must be in [0, {total}), got {start}.")
    if k == 0 or k == total:
        return torch.arange(k, device=device)
    if start is None:
        rd = generator.device if generator is not None else device
        start = int(torch.randint(0, total, (1,), generator=generator, device=rd))
    idx = (torch.arange(k, device=device) + start) % total
    return torch.sort(idx).values
