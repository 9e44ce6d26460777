"""Index sampling from a (weighted) population without the 2²⁴-category limit of ``torch.multinomial``.

Parity: ``physicsnemo/nn/functional/weighted_multinomial.py`` — ``weighted_multinomial(input, num_samples,
replacement=False, *, generator=None, strategy="exact", device=None)``; ``input`` is a population size or a 1-D weight
tensor.  Without replacement the exact strategy draws Efraimidis–Spirakis keys ``Exp(1)/w`` and keeps the smallest
(chunked top-k, so memory stays bounded); ``"poisson_gap"`` places samples by normalised exponential gaps (sorted,
one pass, approximately uniform — meant for very large uniform populations).
"""
from typing import Literal

import torch

from ...core.function_spec import FunctionSpec

SamplingStrategy = Literal["exact", "poisson_gap"]
_CHUNK = 1 << 22
_RANDPERM_LIMIT = 1 << 24


def _exact(n: int, k: int, weights, device, generator) -> torch.Tensor:
    if weights is None and n <= _RANDPERM_LIMIT:
        return torch.randperm(n, device=device, generator=generator)[:k]
    dtype = weights.dtype if weights is not None else torch.get_default_dtype()
    best_keys, best_idx = [], []
    for lo in range(0, n, _CHUNK):
        hi = min(lo + _CHUNK, n)
        keys = torch.empty(hi - lo, dtype=dtype, device=device).exponential_(generator=generator)
        if weights is not None:
            w = weights[lo:hi]
            keys.div_(w).masked_fill_(w == 0, torch.inf)
        kk, ii = torch.topk(keys, min(k, hi - lo), largest=False, sorted=True)
        best_keys.append(kk)
        best_idx.append(ii + lo)
    if len(best_keys) == 1:
        return best_idx[0]
    keys, idx = torch.cat(best_keys), torch.cat(best_idx)
    return idx[torch.topk(keys, k, largest=False, sorted=True).indices]


def _poisson_gap(n: int, k: int, device, generator) -> torch.Tensor:
    if k == n:
        return torch.arange(n, device=device)
    gaps = torch.empty(k, device=device, dtype=torch.float64).exponential_(generator=generator)
    gaps = gaps * ((n - k) / gaps.sum()) + 1.0
    pos = torch.cumsum(gaps, dim=0) - gaps[0]
    return pos.floor().long().clamp_(0, n - 1)


def _weighted_multinomial(input, num_samples, replacement=False, *, generator=None, strategy="exact", device=None):
    if not isinstance(num_samples, int) or isinstance(num_samples, bool):
        raise TypeError(f"num_samples must be an int, got {type(num_samples).__name__}.")
    if num_samples < 0:
        raise ValueError(f"num_samples must be non-negative, got {num_samples}.")
    if not isinstance(replacement, bool):
        raise TypeError(f"replacement must be a bool, got {type(replacement).__name__}.")
    if strategy not in ("exact", "poisson_gap"):
        raise ValueError(f"strategy must be 'exact' or 'poisson_gap', got {strategy!r}.")
    want = torch.device(device) if device is not None else None
    if isinstance(input, torch.Tensor):
        w = input
        if w.ndim != 1:
            raise ValueError(f"input weights must be 1D, got {w.ndim}D with {w.shape=}.")
        if not w.is_floating_point():
            raise TypeError(f"input weights must be floating point, got {w.dtype=}.")
        if not bool(torch.isfinite(w).all()) or bool((w < 0).any()):
            raise RuntimeError("input weights must contain only finite, non-negative values.")
        positive = int(torch.count_nonzero(w > 0))
        if num_samples and positive == 0:
            raise RuntimeError("input weights must contain at least one positive value.")
        if not replacement and num_samples > positive:
            raise RuntimeError("cannot sample more indices than positive input weights without replacement, got "
                               f"{num_samples=} and positive_count={positive}.")
        if strategy == "poisson_gap":
            raise ValueError("poisson_gap sampling requires an integer uniform population.")
        if want is not None and want != w.device:
            raise ValueError(f"device must match input.device when weights are supplied, got {want} and {w.device}.")
        n, dev = w.shape[0], w.device
    elif isinstance(input, int) and not isinstance(input, bool):
        w, n = None, input
        if n < 0:
            raise ValueError(f"input population size must be non-negative, got {input}.")
        if not replacement and num_samples > n:
            raise ValueError("num_samples cannot exceed the input population size without replacement, got "
                             f"{num_samples=} and population_size={n}.")
        if replacement and num_samples and n == 0:
            raise ValueError("cannot sample from an empty input population with replacement.")
        dev = want or torch.device("cpu")
    else:
        raise TypeError(f"input must be an integer population size or a torch.Tensor of weights, got {type(input).__name__}.")
    if strategy == "poisson_gap" and replacement:
        raise ValueError("poisson_gap sampling does not support replacement.")
    if generator is not None and torch.device(generator.device).type != dev.type:
        raise ValueError(f"generator.device must match the sampling device, got {generator.device} and {dev}.")
    if num_samples == 0:
        return torch.empty(0, dtype=torch.long, device=dev)
    if replacement:
        if w is None:
            return torch.randint(n, (num_samples,), device=dev, generator=generator)
        return torch.multinomial(w, num_samples, replacement=True, generator=generator)
    if strategy == "poisson_gap":
        return _poisson_gap(n, num_samples, dev, generator)
    return _exact(n, num_samples, w, dev, generator)


class WeightedMultinomial(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(input, num_samples, replacement=False, *, generator=None, strategy="exact", device=None):
        return _weighted_multinomial(input, num_samples, replacement, generator=generator, strategy=strategy, device=device)


weighted_multinomial = WeightedMultinomial.make_function("weighted_multinomial")
