"""Index helpers shared by readers and sub-sampling transforms (parity: ``physicsnemo/datapipes/_indexing.py``)."""
from __future__ import annotations

from typing import Optional

import torch


def _check_block_request(total: int, k: int, start: Optional[int], has_generator: bool) -> None:
    problems = []
    if min(total, k) < 0:
        problems.append(f"sizes cannot be negative (total={total}, k={k})")
    elif k > total:
        problems.append(f"a block of {k} does not fit into a range of {total}")
    if start is not None:
        if has_generator:
            problems.append("give either a start position or a generator, not both")
        if not (0 <= start < max(total, 1)):
            problems.append(f"start={start} lies outside [0, {total})")
    if problems:
        raise ValueError("; ".join(problems))


def _cyclic_block_indices(total: int, k: int, start: int | None = None, device=None, *,
                          generator: torch.Generator | None = None) -> torch.Tensor:
    """``k`` consecutive indices of ``[0, total)`` starting at a uniformly random (or given) position and wrapping at
    the end: every element is included with probability exactly ``k / total`` while the selection stays one or two
    contiguous runs (friendly to memory-mapped and chunked stores).  Returned in ascending order."""
    _check_block_request(total, k, start, generator is not None)
    if k in (0, total):                                   # nothing to choose
        return torch.arange(k, device=device)
    if start is None:
        draw_on = device if generator is None else generator.device
        start = torch.randint(0, total, (1,), generator=generator, device=draw_on).item()
    first = int(start)
    tail = min(k, total - first)                          # run first .. first + tail - 1, then the wrapped head
    head = k - tail
    pieces = [torch.arange(head, device=device), torch.arange(first, first + tail, device=device)]
    return torch.cat(pieces)
