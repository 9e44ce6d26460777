"""Patch-based ("multi-diffusion") wrapper of a 2-D diffusion model for domains too large to process at once.

Parity: ``physicsnemo/diffusion/multi_diffusion/models.py`` (``MultiDiffusionModel2D``): the wrapped model always sees
patches ``[P·B, C, Hp, Wp]``; ``x``, ``t`` and the condition are patched on the way in (random patches for training, a
regular overlapping grid for inference), an optional positional embedding of the *global* grid is patched alike and handed
to the model inside the condition, and grid patches can be fused back by overlap-averaging.

Conditions are a tensor, ``None`` or a mapping of named tensors; the reference uses ``tensordict.TensorDict`` for the
latter, this implementation returns the small ``ConditionDict`` (a ``dict`` with a ``batch_size`` and batch slicing) so no
extra dependency is needed.  Mapping conditions take per-key ``condition_patch`` / ``condition_interp`` flags: patch the
tensor like ``x``, bilinearly resize it to the patch size, or just repeat it for every patch.
"""
from __future__ import annotations

import math
import warnings
from collections import defaultdict
from typing import Any, Dict, Literal, Mapping, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from ...core.module import Module
from .patching import GridPatching2D, RandomPatching2D


class ConditionDict(dict):
    """Named condition tensors sharing a leading batch axis; ``cond[a:b]`` slices every entry."""

    def __init__(self, data: Mapping[str, Tensor] | None = None, batch_size=None):
        super().__init__(data or {})
        self.batch_size = list(batch_size) if batch_size is not None else ([next(iter(self.values())).shape[0]] if self else [0])

    def __getitem__(self, key):
        if isinstance(key, slice):
            out = ConditionDict({k: v[key] for k, v in self.items()})
            out.batch_size = [len(range(*key.indices(self.batch_size[0])))]
            return out
        return super().__getitem__(key)

    def to(self, *args, **kwargs) -> "ConditionDict":
        return ConditionDict({k: v.to(*args, **kwargs) for k, v in self.items()}, self.batch_size)


def _is_mapping(c) -> bool:
    return isinstance(c, Mapping) or (hasattr(c, "keys") and hasattr(c, "__getitem__") and not isinstance(c, Tensor))


class MultiDiffusionModel2D(Module):
    def __init__(self, model: torch.nn.Module, global_spatial_shape: Tuple[int, int],
                 positional_embedding: Literal["learnable", "sinusoidal", "linear"] | None = None, channels_positional_embedding: int = 4,
                 condition_patch: bool | Dict[str, bool] = False, condition_interp: bool | Dict[str, bool] = False):
        super().__init__()
        self.model = model
        self.global_spatial_shape = tuple(global_spatial_shape)
        self._patching: RandomPatching2D | GridPatching2D | None = None
        self._fuse = False
        self._skip_positional_embedding_injection = False
        self.register_buffer("_patch_shape", torch.zeros(2, dtype=torch.long), persistent=True)
        for name, v in (("condition_patch", condition_patch), ("condition_interp", condition_interp)):
            if not isinstance(v, (bool, dict)):
                raise TypeError(f"{name} must be bool or Dict[str, bool], got {type(v).__name__}.")
        self._condition_has_per_key_flags = isinstance(condition_patch, dict) or isinstance(condition_interp, dict)
        mk = lambda v: defaultdict(lambda: v) if isinstance(v, bool) else defaultdict(lambda: False, v)  # noqa: E731
        self._condition_patch, self._condition_interp = mk(condition_patch), mk(condition_interp)
        H, W = self.global_spatial_shape
        C = channels_positional_embedding
        if positional_embedding is None:
            self.pos_embd = None
        elif positional_embedding == "learnable":
            self.pos_embd = torch.nn.Parameter(torch.randn(C, H, W))
        elif positional_embedding == "linear":
            if C != 2:
                raise ValueError("a linear positional embedding has exactly 2 channels")
            gy, gx = torch.meshgrid(torch.linspace(-1, 1, H), torch.linspace(-1, 1, W), indexing="ij")
            self.register_buffer("pos_embd", torch.stack([gy, gx]))
        elif positional_embedding == "sinusoidal":
            if C % 4:
                raise ValueError("a sinusoidal positional embedding needs a channel count divisible by 4")
            gy, gx = torch.meshgrid(torch.linspace(0, 2 * math.pi, H), torch.linspace(0, 2 * math.pi, W), indexing="ij")
            maps = []
            for k in range(C // 4):
                for fn in (torch.sin, torch.cos):
                    maps += [fn(gx * 2.0 ** k), fn(gy * 2.0 ** k)]
            self.register_buffer("pos_embd", torch.stack(maps), persistent=False)
        else:
            raise ValueError(f"unknown positional_embedding {positional_embedding!r}")

    # ---- patching set-up
    @property
    def condition_patch(self):
        return self._condition_patch

    @property
    def condition_interp(self):
        return self._condition_interp

    @property
    def patch_shape(self) -> tuple[int, int] | None:
        if self._patching is not None:
            return tuple(self._patching.patch_shape)
        ps = self._patch_shape
        return (int(ps[0]), int(ps[1])) if int(ps[0]) > 0 or int(ps[1]) > 0 else None

    def _remember(self, patch_shape):
        self._patch_shape[0], self._patch_shape[1] = int(patch_shape[0]), int(patch_shape[1])

    def set_random_patching(self, patch_shape: Tuple[int, int], patch_num: int) -> None:
        self._patching = RandomPatching2D(img_shape=self.global_spatial_shape, patch_shape=patch_shape, patch_num=patch_num)
        self._fuse = False
        self._remember(patch_shape)

    def reset_patch_indices(self) -> None:
        if not isinstance(self._patching, RandomPatching2D):
            raise RuntimeError("reset_patch_indices() is only available when random patching is active. Call set_random_patching() first.")
        self._patching.reset_patch_indices()

    def set_grid_patching(self, patch_shape: Tuple[int, int], overlap_pix: int = 0, boundary_pix: int = 0, fuse: bool = True) -> None:
        self._patching = GridPatching2D(img_shape=self.global_spatial_shape, patch_shape=patch_shape, overlap_pix=overlap_pix, boundary_pix=boundary_pix)
        self._fuse = fuse
        self._remember(patch_shape)

    def _need_patching(self):
        if self._patching is None:
            raise RuntimeError("No patching strategy set. Call set_random_patching() or set_grid_patching() first.")
        return self._patching

    # ---- patch / fuse primitives
    def patch_x(self, x: Tensor) -> Tensor:
        patching = self._need_patching()
        if x.ndim != 4 or tuple(x.shape[2:]) != self.global_spatial_shape:
            raise ValueError(f"expected x of shape (B, C, {self.global_spatial_shape[0]}, {self.global_spatial_shape[1]}), got {tuple(x.shape)}")
        return patching.apply(x)

    def patch_t(self, t: Tensor) -> Tensor:
        return t.repeat(self._need_patching().patch_num)

    def _process_condition_tensor(self, tensor: Tensor, do_patch: bool, do_interp: bool, P: int) -> Tensor:
        if do_patch and do_interp:
            raise ValueError("a condition cannot be both patched and interpolated")
        if (do_patch or do_interp) and tensor.ndim != 4:
            raise ValueError(f"patched / interpolated conditions must be (B, C, H, W), got {tuple(tensor.shape)}")
        if not do_patch and not do_interp:
            return tensor.repeat(P, *[1] * (tensor.ndim - 1))
        patching = self._need_patching()
        if do_patch:
            if tuple(tensor.shape[2:]) != self.global_spatial_shape:
                raise ValueError(f"a patched condition must have the global spatial shape {self.global_spatial_shape}, got {tuple(tensor.shape[2:])}")
            return patching.apply(tensor)
        return F.interpolate(tensor, size=tuple(patching.patch_shape), mode="bilinear").repeat(P, 1, 1, 1)

    def patch_condition(self, condition):
        P = self._need_patching().patch_num
        if condition is None:
            return None
        if isinstance(condition, Tensor):
            if self._condition_has_per_key_flags:
                raise ValueError("per-key condition flags need a mapping condition")
            return self._process_condition_tensor(condition, self._condition_patch[""], self._condition_interp[""], P)
        if _is_mapping(condition):
            keys = set(condition.keys())
            for flags, name in ((self._condition_patch, "condition_patch"), (self._condition_interp, "condition_interp")):
                extra = set(flags) - keys
                if extra:
                    raise ValueError(f"{name} names keys that the condition does not have: {sorted(extra)}")
            B = next(iter(condition.values())).shape[0] if not hasattr(condition, "batch_size") else list(condition.batch_size)[0]
            return ConditionDict({k: self._process_condition_tensor(condition[k], self._condition_patch[k], self._condition_interp[k], P)
                                  for k in condition.keys()}, batch_size=[P * B])
        raise TypeError(f"condition must be Tensor, a mapping of tensors, or None, got {type(condition).__name__}.")

    def fuse(self, input: Tensor, batch_size: int) -> Tensor:
        if not isinstance(self._patching, GridPatching2D):
            raise RuntimeError("Fusing is only supported with grid patching. Call set_grid_patching() first.")
        return self._patching.fuse(input, batch_size=batch_size)

    @staticmethod
    def _inject_patched_pos_embd(condition, pos_embd_patched: Tensor, PB: int) -> ConditionDict:
        if condition is None:
            return ConditionDict({"positional_embedding": pos_embd_patched}, batch_size=[PB])
        if isinstance(condition, Tensor):
            return ConditionDict({"condition": condition, "positional_embedding": pos_embd_patched}, batch_size=[PB])
        out = condition if isinstance(condition, ConditionDict) else ConditionDict(dict(condition), batch_size=[PB])
        out["positional_embedding"] = pos_embd_patched
        return out

    def forward(self, x: Tensor, t: Tensor, condition=None, x_is_patched: bool = False, t_is_patched: bool = False,
                condition_is_patched: bool = False, **model_kwargs: Any) -> Tensor:
        patching = self._patching
        inject = self.pos_embd is not None and not self._skip_positional_embedding_injection
        if patching is None:
            warnings.warn("No patching strategy set on MultiDiffusionModel2D. The model will run without patching.", stacklevel=2)
            if inject:
                B = x.shape[0]
                condition = self._inject_patched_pos_embd(condition, self.pos_embd.unsqueeze(0).expand(B, -1, -1, -1).contiguous(), B)
            return self.model(x, t, condition=condition, **model_kwargs)
        P = patching.patch_num
        needs_b = inject or self._fuse
        if x_is_patched:
            if needs_b and x.shape[0] % P:
                raise ValueError(f"the patched batch {x.shape[0]} is not a multiple of the patch count {P}")
            B = x.shape[0] // P if needs_b else 0
        else:
            B = x.shape[0]
            x = self.patch_x(x)
        if not t_is_patched:
            t = self.patch_t(t)
        if not condition_is_patched:
            condition = self.patch_condition(condition)
        if inject:
            pe = patching.apply(self.pos_embd.unsqueeze(0).expand(B, -1, -1, -1).contiguous())
            condition = self._inject_patched_pos_embd(condition, pe, P * B)
        out = self.model(x, t, condition=condition, **model_kwargs)
        return patching.fuse(out, batch_size=B) if self._fuse else out
