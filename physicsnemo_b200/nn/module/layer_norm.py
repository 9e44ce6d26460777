"""LayerNorm class selection.

Parity: ``physicsnemo/nn/module/layer_norm.py:88-164`` (``get_layer_norm_class`` and the
exported ``LayerNorm``).  The reference picks Transformer-Engine's fused LayerNorm when it
is installed; here ``LayerNorm`` is a ``torch.nn.LayerNorm`` subclass (same ``weight`` /
``bias`` keys) whose CUDA bf16 forward/backward run on the library's warp-per-row kernels.
Checkpoints written by a Transformer-Engine build carry ``_extra_state`` entries, which are
dropped on load like the reference does (``:29-85``).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops


def _drop_te_extra_state(module, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
    key = prefix + "_extra_state"
    if key in state_dict:
        state_dict.pop(key)


class LayerNorm(nn.LayerNorm):
    """``torch.nn.LayerNorm`` with the fused sm_100a kernels on CUDA bf16 inputs."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._register_load_state_dict_pre_hook(_drop_te_extra_state, with_module=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if (
            len(self.normalized_shape) == 1
            and self.weight is not None
            and ops.fused_path_enabled(x)
        ):
            return ops.layer_norm(x, self.weight, self.bias, self.eps)
        return super().forward(x)


def get_layer_norm_class():
    """Return the LayerNorm class used across the package."""
    return LayerNorm


def remove_extra_state_hook_for_torch(module, state_dict, prefix, local_metadata):
    """State-dict hook kept for API parity: nothing to strip for the torch-based class."""
    return state_dict
