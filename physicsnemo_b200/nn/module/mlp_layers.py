"""Generic MLP (``Linear → act → … → Linear``).

Parity: ``physicsnemo/nn/module/mlp_layers.py:32-173`` — parameters live under
``layers.<i>`` of an ``nn.Sequential``; the activation sits between linears,
optional BatchNorm / dropout / spectral norm.  On CUDA bf16/fp16 inputs every
``Linear(+activation)`` pair runs as one tcgen05 GEMM with the bias and the
activation applied in the epilogue (``physicsnemo_b200.ops.linear``).
"""
from __future__ import annotations

import itertools

import torch
import torch.nn as nn

from .activations import activation_code, get_activation
from ... import ops


class Mlp(nn.Module):
    def __init__(
        self,
        in_features: int,
        hidden_features: int | list[int] | None = None,
        out_features: int | None = None,
        act_layer: nn.Module | type[nn.Module] | str = nn.GELU,
        drop: float = 0.0,
        final_dropout: bool = True,
        bias: bool = True,
        use_batchnorm: bool = False,
        spectral_norm: bool = False,
        use_te: bool = False,
    ):
        super().__init__()
        # ``use_te`` is accepted for signature parity; the fused kernels here
        # replace Transformer-Engine and keep the plain ``nn.Linear`` key names.
        self.use_te = False
        out_features = out_features or in_features
        if hidden_features is None:
            hidden_features = [in_features]
        elif isinstance(hidden_features, int):
            hidden_features = [hidden_features]
        if isinstance(act_layer, str):
            act_layer = get_activation(act_layer)
        elif not isinstance(act_layer, nn.Module):
            act_layer = act_layer()
            if not isinstance(act_layer, nn.Module):
                raise ValueError(f"Activation layer must be a string or a module, got {type(act_layer)}")
        layers: list[nn.Module] = []
        dims = [in_features, *hidden_features, out_features]
        n_layers = len(dims) - 1
        for i, (d_in, d_out) in enumerate(itertools.pairwise(dims)):
            last = i == n_layers - 1
            linear = nn.Linear(d_in, d_out, bias=bias)
            if spectral_norm:
                linear = nn.utils.parametrizations.spectral_norm(linear, name="weight")
            layers.append(linear)
            if use_batchnorm:
                layers.append(nn.BatchNorm1d(d_out))
            if not last:
                layers.append(act_layer)
            if drop != 0 and (not last or final_dropout):
                layers.append(nn.Dropout(drop))
        self.layers = nn.Sequential(*layers)
        self._fusable = not (use_batchnorm or spectral_norm)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not (self._fusable and ops.fused_path_enabled(x)):
            return self.layers(x)
        # maximal runs of Linear(+activation) go through one fused chain, so that the activation
        # derivative is applied inside the next layer's input-gradient GEMM
        mods = list(self.layers)
        i = 0
        ws, bs, acts = [], [], []

        def flush(h):
            if ws:
                h = ops.mlp_chain(h, list(ws), list(bs), list(acts))
                ws.clear(), bs.clear(), acts.clear()
            return h

        while i < len(mods):
            m = mods[i]
            if isinstance(m, nn.Linear):
                code = 0
                if i + 1 < len(mods) and not isinstance(mods[i + 1], (nn.Dropout, nn.Linear)):
                    c = activation_code(mods[i + 1])
                    if c:
                        code = c
                ws.append(m.weight), bs.append(m.bias), acts.append(code)
                i += 2 if code else 1
            else:
                x = m(flush(x))
                i += 1
        return flush(x)
