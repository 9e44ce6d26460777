"""Out-of-distribution guard embedded in a GeoTransolver.

Counterpart of ``physicsnemo/experimental/guardrails/embedded/geotransolver_guard.py`` (``GuardedGeoTransolver`` :58,
``attach_ood_guard`` :348).  The wrapper watches two surfaces of the wrapped model: the raw global embedding (per-channel
range seen in training) and the geometry latent (mean over heads and slices of the geometry tokenizer's output, captured
by a forward hook; kNN distance against a buffer of training latents).  In training mode the guard collects, in
evaluation mode it checks and warns; the model's output is returned unchanged.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .ood_guard import OODGuard, OODGuardConfig

__all__ = ["GuardedGeoTransolver", "attach_ood_guard"]


def _geometry_embed_dim(model: nn.Module) -> Optional[int]:
    tok = getattr(model.context_builder, "geometry_tokenizer", None)
    return None if tok is None else int(tok.dim_head)


def _global_dim(model: nn.Module) -> Optional[int]:
    tok = getattr(model.context_builder, "global_tokenizer", None)
    return None if tok is None else int(tok.in_project_x.in_features)


def _as_tuple(t):
    return (t,) if isinstance(t, torch.Tensor) else tuple(t)


class GuardedGeoTransolver(nn.Module):
    def __init__(self, model: nn.Module, config: OODGuardConfig, *, global_dim: Optional[int] = None,
                 geometry_embed_dim: Optional[int] = None):
        super().__init__()
        global_dim = _global_dim(model) if global_dim is None else global_dim
        geometry_embed_dim = _geometry_embed_dim(model) if geometry_embed_dim is None else geometry_embed_dim
        if global_dim is None and geometry_embed_dim is None:
            raise ValueError("GuardedGeoTransolver requires the wrapped model to enable at least one of the global or geometry "
                             "surfaces; both are disabled, so the OOD guard would have nothing to watch.")
        self.model = model
        self.ood_guard = OODGuard(buffer_size=config.buffer_size, global_dim=global_dim, geometry_embed_dim=geometry_embed_dim,
                                  knn_k=config.knn_k, sensitivity=config.sensitivity)
        self._geo_latent: Optional[torch.Tensor] = None
        tok = getattr(model.context_builder, "geometry_tokenizer", None)
        self._geo_hook_handle = None if tok is None else tok.register_forward_hook(self._capture)

    def _capture(self, module, inputs, output) -> None:
        self._geo_latent = output.detach().mean(dim=(1, 2))            # [B, heads, slices, head_dim] -> [B, head_dim]

    def _validate(self, local_embedding, local_positions, global_embedding, geometry) -> None:
        locals_ = _as_tuple(local_embedding)
        if not locals_:
            raise ValueError("Expected non-empty local_embedding")
        ranks = {3}
        shape = getattr(self.model, "structured_shape", None)
        if shape is not None:
            ranks.add(len(shape) + 2)
        want = " or ".join(f"{r}D" for r in sorted(ranks))
        for i, t in enumerate(locals_):
            if t.ndim not in ranks:
                raise ValueError(f"Expected {want} local_embedding tensor at index {i} but got tensor of shape {tuple(t.shape)}")
        if local_positions is not None:
            for i, t in enumerate(_as_tuple(local_positions)):
                if t.ndim != 3:
                    raise ValueError(f"Expected local_positions tensor of shape (B, N, D_p) at index {i} but got tensor of shape "
                                     f"{tuple(t.shape)}")
        if global_embedding is not None:
            if global_embedding.ndim != 3:
                raise ValueError(f"Expected global_embedding tensor of shape (B, N_g, C_g) but got tensor of shape "
                                 f"{tuple(global_embedding.shape)}")
            gm = self.ood_guard.global_min
            if gm is not None and global_embedding.shape[-1] != gm.shape[0]:
                raise ValueError(f"Expected global_embedding tensor of shape (B, N_g, {gm.shape[0]}) but got tensor of shape "
                                 f"{tuple(global_embedding.shape)}")
        if geometry is not None and geometry.ndim not in ranks:
            raise ValueError(f"Expected {want} geometry tensor but got tensor of shape {tuple(geometry.shape)}")

    def forward(self, local_embedding, local_positions=None, global_embedding=None, geometry=None, time=None,
                return_embedding_states: bool = False):
        if not torch.compiler.is_compiling():
            self._validate(local_embedding, local_positions, global_embedding, geometry)
        self._geo_latent = None
        out = self.model(local_embedding, local_positions=local_positions, global_embedding=global_embedding, geometry=geometry, time=time,
                         return_embedding_states=return_embedding_states)
        (self.ood_guard.collect if self.model.training else self.ood_guard.check)(global_embedding, self._geo_latent)
        return out

    def close(self) -> None:
        """Remove the forward hook from the wrapped model."""
        if self._geo_hook_handle is not None:
            self._geo_hook_handle.remove()
            self._geo_hook_handle = None


def attach_ood_guard(model: nn.Module, config: OODGuardConfig, *, global_dim: Optional[int] = None,
                     geometry_embed_dim: Optional[int] = None) -> GuardedGeoTransolver:
    return GuardedGeoTransolver(model, config, global_dim=global_dim, geometry_embed_dim=geometry_embed_dim)
