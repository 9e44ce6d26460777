"""Diffusion posterior sampling guidance evaluated patch by patch on multi-diffusion domains.

Parity: ``physicsnemo/diffusion/multi_diffusion/dps_guidance.py`` — ``MultiDiffusionDPSGuidance`` (protocol),
``MultiDiffusionDPSScorePredictor``, ``MultiDiffusionModelConsistencyDPSGuidance`` and
``MultiDiffusionDataConsistencyDPSGuidance``.  A guidance is *patch-local* when its value on a patch depends only on
that patch's data.  Observations, their uncertainties and masks are cut into the predictor's patch layout once, at
construction; a call then receives a chunk of ``K`` patches (``slice_start`` names the chunk's first row in the
``P·B`` patch batch) and differentiates only through that chunk's network evaluation, so peak memory follows the chunk
size instead of the number of patches.  The score predictor streams ``score + Σ guidance`` chunk by chunk and fuses
the patches once at the end.
"""
from __future__ import annotations

from typing import Callable, Optional, Protocol, Sequence, Union, runtime_checkable

import torch
from torch import Tensor

from ..guidance.dps_guidance import _as_broadcastable, _needs_autograd
from .predictor import MultiDiffusionPredictor


@runtime_checkable
class MultiDiffusionDPSGuidance(Protocol):
    """``guidance(x, t, x_0, slice_start=None) -> Tensor`` on ``[K, C, Hp, Wp]`` patch batches.  ``slice_start=None``: the
    whole ``P·B`` batch at once; an integer: the chunk of ``K`` patches that starts at that row."""

    def __call__(self, x: Tensor, t: Tensor, x_0: Tensor, slice_start: Optional[int] = None) -> Tensor: ...


def _patch_like(value, predictor: MultiDiffusionPredictor, y: Tensor) -> Tensor:
    """``value`` (scalar or broadcastable to the global observation ``y``) in the predictor's patch layout."""
    full = torch.broadcast_to(_as_broadcastable(value, y), y.shape).contiguous()
    return predictor.patch_fn(full)


class MultiDiffusionDPSScorePredictor:
    """``Fuse[ score(x̂₀ᵏ, xᵏ, tᵏ) + Σᵢ gᵢ(xᵏ, tᵏ, x̂₀ᵏ) ]`` over the chunks ``k`` of the patch batch.

    ``x0_predictor`` must be a ``MultiDiffusionPredictor`` built with a ``chunk_size``; ``x0_to_score_fn(x_0, x_t, t)`` is
    an element-wise conversion (e.g. a noise scheduler's ``x0_to_score``).  Call under ``torch.no_grad()`` in sampling
    loops (autograd is re-enabled inside for the guidances); ``torch.inference_mode()`` is rejected."""

    def __init__(self, x0_predictor: MultiDiffusionPredictor, x0_to_score_fn: Callable[[Tensor, Tensor, Tensor], Tensor],
                 guidances: Union[MultiDiffusionDPSGuidance, Sequence[MultiDiffusionDPSGuidance]]) -> None:
        if not isinstance(x0_predictor, MultiDiffusionPredictor):
            raise TypeError(f"a MultiDiffusionPredictor is required, got {type(x0_predictor).__name__}")
        if x0_predictor._chunk_size is None:
            raise ValueError("the MultiDiffusionPredictor must be built with chunk_size=<int>: guidance is evaluated chunk by chunk")
        self.x0_predictor, self.x0_to_score_fn = x0_predictor, x0_to_score_fn
        many = isinstance(guidances, Sequence) and not isinstance(guidances, str)
        self.guidances = list(guidances) if many else [guidances]

    def __call__(self, x: Tensor, t: Tensor) -> Tensor:
        _needs_autograd("MultiDiffusionDPSScorePredictor")
        keep_graph = torch.is_grad_enabled()
        x = x.detach().requires_grad_(True)
        pieces = []
        with torch.enable_grad():
            for start, x0_chunk, x_chunk, t_chunk in self.x0_predictor.chunks(x, t):
                pull = torch.zeros_like(x0_chunk)
                for guidance in self.guidances:
                    pull = pull + guidance(x_chunk, t_chunk, x0_chunk, slice_start=start)
                with torch.set_grad_enabled(keep_graph):       # under no_grad the pieces are leaves: no graph accumulates
                    pieces.append(self.x0_to_score_fn(x0_chunk, x_chunk, t_chunk) + pull)
        return self.x0_predictor.fuse_fn(torch.cat(pieces, dim=0))


class _PatchLocalConsistency:
    """Shared part of the two guidances: ``−∇ₓ Σ ρ(t) · loss`` with ``ρ = 1 / (2 (σ_y² + γ σ(t)² / α(t)²))``."""

    def __init__(self, predictor: MultiDiffusionPredictor, y: Tensor, std_y, norm, gamma, sigma_fn, alpha_fn, fuse, retain_graph,
                 create_graph) -> None:
        self.predictor = predictor
        self._y_patched = predictor.patch_fn(y)
        self._std_y_patched = _patch_like(std_y, predictor, y)
        self._gamma_patched = _patch_like(gamma, predictor, y)
        if sigma_fn is None and bool((self._gamma_patched > 0).any()):
            raise ValueError("gamma > 0 needs sigma_fn (the noise level as a function of time)")
        self._loss_fn = (lambda a, b, p=norm: (a - b).abs().pow(p)) if isinstance(norm, int) else norm
        self.sigma_fn = sigma_fn if sigma_fn is not None else torch.zeros_like
        self.alpha_fn = alpha_fn if alpha_fn is not None else torch.ones_like
        self.fuse, self.retain_graph, self.create_graph = fuse, retain_graph, create_graph

    def _chunk(self, stored: Tensor, rows: slice, like: Tensor) -> Tensor:
        return stored[rows].to(dtype=like.dtype, device=like.device)

    def _loss(self, x_0: Tensor, rows: slice) -> Tensor:
        raise NotImplementedError

    def __call__(self, x: Tensor, t: Tensor, x_0: Tensor, slice_start: Optional[int] = None) -> Tensor:
        _needs_autograd(type(self).__name__)
        rows = slice(None) if slice_start is None else slice(slice_start, slice_start + x.shape[0])
        with torch.enable_grad():
            loss = self._loss(x_0, rows)
            t_b = t.reshape((-1,) + (1,) * (loss.ndim - 1))
            spread = self._chunk(self._std_y_patched, rows, x) ** 2 + self._chunk(self._gamma_patched, rows, x) * (
                self.sigma_fn(t_b) ** 2 / self.alpha_fn(t_b) ** 2)
            objective = (loss / (2.0 * spread)).sum()
            grad = torch.autograd.grad(objective, x, retain_graph=self.retain_graph, create_graph=self.create_graph)[0]
        pull = -grad
        return self.predictor.fuse_fn(pull) if (slice_start is None and self.fuse) else pull


class MultiDiffusionModelConsistencyDPSGuidance(_PatchLocalConsistency):
    """Towards observations ``y ≈ A(x₀)`` of a differentiable, patch-local observation operator ``A`` (applied per patch)."""

    def __init__(self, predictor: MultiDiffusionPredictor, observation_operator: Callable[[Tensor], Tensor], y: Tensor, std_y,
                 norm=2, gamma=0.0, sigma_fn=None, alpha_fn=None, fuse: bool = False, retain_graph: bool = False,
                 create_graph: bool = False) -> None:
        super().__init__(predictor, y, std_y, norm, gamma, sigma_fn, alpha_fn, fuse, retain_graph, create_graph)
        self.observation_operator = observation_operator

    def _loss(self, x_0, rows):
        return self._loss_fn(self.observation_operator(x_0), self._chunk(self._y_patched, rows, x_0))


class MultiDiffusionDataConsistencyDPSGuidance(_PatchLocalConsistency):
    """Towards observations of the state itself where ``mask`` is set (in-painting, sparse sensors)."""

    def __init__(self, predictor: MultiDiffusionPredictor, mask: Tensor, y: Tensor, std_y, norm=2, gamma=0.0, sigma_fn=None,
                 alpha_fn=None, fuse: bool = False, retain_graph: bool = False, create_graph: bool = False) -> None:
        super().__init__(predictor, y, std_y, norm, gamma, sigma_fn, alpha_fn, fuse, retain_graph, create_graph)
        self._mask_patched = predictor.patch_fn(torch.broadcast_to(mask.to(y.dtype), y.shape).contiguous())

    def _loss(self, x_0, rows):
        return self._chunk(self._mask_patched, rows, x_0) * self._loss_fn(x_0, self._chunk(self._y_patched, rows, x_0))
