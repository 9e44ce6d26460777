"""Inference-time ``x0`` predictor over a regular patch grid, with optional chunking and activation checkpointing.

Parity: ``physicsnemo/diffusion/multi_diffusion/predictor.py`` (``MultiDiffusionPredictor``): the condition and the
positional embedding are patched once in ``set_patching``; every call patches ``x`` and ``t``, runs the wrapped model on
all patches (or ``chunk_size`` patches at a time), converts to ``x0`` and overlap-averages the patches back to the global
grid unless ``fuse`` is off.
"""
from __future__ import annotations

import warnings
from typing import Any, Iterator

import torch
from torch import Tensor
from torch.utils.checkpoint import checkpoint

from .losses import _unwrap_module, _x0_converter
from .models import MultiDiffusionModel2D


class MultiDiffusionPredictor:
    def __init__(self, model, condition=None, fuse: bool = True, chunk_size: int | None = None, use_checkpointing: bool = False,
                 prediction_type: str = "x0", score_to_x0_fn=None, epsilon_to_x0_fn=None, **model_kwargs: Any):
        self._md_model: MultiDiffusionModel2D = _unwrap_module(model, MultiDiffusionModel2D)
        self.model, self._model_kwargs = model, model_kwargs
        self._chunk_size, self._use_checkpointing, self._fuse = chunk_size, use_checkpointing, fuse
        self._cond_input = condition
        self._patch_shape = self._md_model.patch_shape
        self._global_shape = tuple(self._md_model.global_spatial_shape)
        self._patching, self._P, self._cond_patched, self._pos_embd_patched = None, None, None, None
        self._md_model._skip_positional_embedding_injection = True       # this class injects the pre-patched embedding itself
        self._md_model._fuse = False
        self._to_x0 = _x0_converter(prediction_type, score_to_x0_fn, epsilon_to_x0_fn)

    @property
    def fuse(self) -> bool:
        return self._fuse

    @fuse.setter
    def fuse(self, value: bool) -> None:
        self._fuse = value

    @property
    def patch_shape(self):
        return self._md_model.patch_shape

    def _check_patching_set(self) -> None:
        if self._patching is None:
            raise RuntimeError("Grid patching is not configured. Call set_patching(overlap_pix, boundary_pix, ...) before any other method.")

    def set_patching(self, overlap_pix: int, boundary_pix: int, *, patch_shape=None, global_shape=None) -> None:
        if patch_shape is not None:
            if self._patch_shape is not None and tuple(patch_shape) != tuple(self._patch_shape):
                warnings.warn(f"Overriding saved patch_shape {self._patch_shape} with {tuple(patch_shape)}. Inference-time patching that "
                              "differs from training may produce unexpected results.", stacklevel=2)
            self._patch_shape = tuple(patch_shape)
        if global_shape is not None:
            if tuple(global_shape) != self._global_shape:
                warnings.warn(f"Overriding saved global_spatial_shape {self._global_shape} with {tuple(global_shape)}. Positional embeddings "
                              "baked at model construction will no longer match the new shape.", stacklevel=2)
            self._global_shape = tuple(global_shape)
        if self._patch_shape is None:
            raise RuntimeError("patch_shape is not available on the wrapped model and was not provided. Pass patch_shape=(Hp, Wp) explicitly.")
        md = self._md_model
        md.global_spatial_shape = self._global_shape
        md.set_grid_patching(patch_shape=self._patch_shape, overlap_pix=overlap_pix, boundary_pix=boundary_pix, fuse=False)
        self._patching, self._P = md._patching, md._patching.patch_num
        self._cond_patched = md.patch_condition(self._cond_input)
        self._pos_embd_patched = md.patch_x(md.pos_embd.unsqueeze(0)) if md.pos_embd is not None else None

    def patch_fn(self, x: Tensor) -> Tensor:
        self._check_patching_set()
        return self._md_model.patch_x(x)

    def fuse_fn(self, patched: Tensor) -> Tensor:
        self._check_patching_set()
        return self._md_model.fuse(patched, batch_size=patched.shape[0] // self._P)

    def _build_cond(self, B: int):
        cond = self._cond_patched
        if self._pos_embd_patched is not None:
            cond = self._md_model._inject_patched_pos_embd(cond, self._pos_embd_patched.repeat_interleave(B, dim=0), self._P * B)
        return cond

    def _call_model(self, x_p: Tensor, t_p: Tensor, cond) -> Tensor:
        run = lambda xc, tc: self._md_model(xc, tc, condition=cond, x_is_patched=True, t_is_patched=True, condition_is_patched=True,  # noqa: E731
                                            **self._model_kwargs)
        return checkpoint(run, x_p, t_p, use_reentrant=False) if self._use_checkpointing else run(x_p, t_p)

    def chunks(self, x: Tensor, t: Tensor) -> Iterator[tuple[int, Tensor, Tensor, Tensor]]:
        """Yield ``(start, x0_chunk, x_chunk, t_chunk)`` over groups of ``chunk_size`` patches."""
        self._check_patching_set()
        if self._chunk_size is None:
            raise RuntimeError("chunk_size must be set at construction to use chunks(). Pass chunk_size=<int> to MultiDiffusionPredictor.__init__.")
        x_p, t_p, cond = self._md_model.patch_x(x), self._md_model.patch_t(t), self._build_cond(x.shape[0])
        for s in range(0, x_p.shape[0], self._chunk_size):
            e = min(s + self._chunk_size, x_p.shape[0])
            xc, tc = x_p[s:e], t_p[s:e]
            out = self._call_model(xc, tc, cond[s:e] if cond is not None else None)
            yield s, self._to_x0(out, xc, tc), xc, tc

    def __call__(self, x: Tensor, t: Tensor) -> Tensor:
        self._check_patching_set()
        if self._chunk_size is not None:
            out = torch.cat([x0_c for _, x0_c, _, _ in self.chunks(x, t)], dim=0)
        else:
            x_p, t_p = self._md_model.patch_x(x), self._md_model.patch_t(t)
            out = self._to_x0(self._call_model(x_p, t_p, self._build_cond(x.shape[0])), x_p, t_p)
        return self.fuse_fn(out) if self._fuse else out
