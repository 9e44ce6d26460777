"""MLPs of MeshGraphNet-style networks.

Parity: ``physicsnemo/nn/module/gnn_layers/mesh_graph_mlp.py`` — ``MeshGraphMLP`` (``:120-206``:
``model`` = Linear, act, (Linear, act)…, Linear, LayerNorm), ``MeshGraphEdgeMLPConcat`` (``:209``),
``MeshGraphHeteroEdgeMLPConcat`` (``:281``), ``MeshGraphEdgeMLPSum`` (``:366-532``: first linear
split into ``lin_efeat / lin_src / lin_dst`` + ``bias``).  The reference's
``recompute_activation`` option trades memory for a recomputed SiLU; here the fused chain
(``ops.mlp_chain``) already keeps only the pre-activations, and the flag is accepted.

Fused path (CUDA, bf16): the whole ``Linear → act → … → Linear`` chain runs on tcgen05 GEMMs
with activations in the epilogues, the K-concatenated edge input ``[efeat | src | dst]`` is
never materialised, and the trailing LayerNorm kernel adds the block's residual.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .... import ops
from ..activations import activation_code
from ..layer_norm import get_layer_norm_class
from .utils import concat_efeat, concat_efeat_hetero, gather_src_dst, sum_efeat


def _chain(model: nn.Sequential, x, post: Optional[Tensor] = None) -> Optional[Tensor]:
    """Run ``model`` (Linear/act…/[LayerNorm]) on the fused kernels; ``None`` if it cannot be fused."""
    mods = list(model)
    norm = mods[-1] if isinstance(mods[-1], nn.LayerNorm) else None
    body = mods[:-1] if norm is not None else mods
    weights, biases, acts = [], [], []
    i = 0
    while i < len(body):
        if not isinstance(body[i], nn.Linear):
            return None
        code = 0
        if i + 1 < len(body) and not isinstance(body[i + 1], nn.Linear):
            code = activation_code(body[i + 1])
            if code is None:
                return None
            i += 1
        weights.append(body[i - (1 if code else 0)].weight)
        biases.append(body[i - (1 if code else 0)].bias)
        acts.append(code)
        i += 1
    if norm is None:
        return ops.mlp_chain(x, weights, biases, acts, residual=post)
    h = ops.mlp_chain(x, weights, biases, acts)
    return ops.layer_norm(h, norm.weight, norm.bias, norm.eps, post=post)


class MeshGraphMLP(nn.Module):
    """``hidden_layers`` hidden Linear+activation layers, an output Linear and an optional LayerNorm."""

    def __init__(self, input_dim: int, output_dim: int = 512, hidden_dim: int = 512,
                 hidden_layers: Union[int, None] = 1, activation_fn: nn.Module = nn.SiLU(),
                 norm_type: str = "LayerNorm", recompute_activation: bool = False):
        super().__init__()
        if hidden_layers is not None:
            layers = [nn.Linear(input_dim, hidden_dim), activation_fn]
            self.hidden_layers = hidden_layers
            for _ in range(hidden_layers - 1):
                layers += [nn.Linear(hidden_dim, hidden_dim), activation_fn]
            layers.append(nn.Linear(hidden_dim, output_dim))
            self.norm_type = norm_type
            if norm_type is not None:
                if norm_type not in ("LayerNorm", "TELayerNorm"):
                    raise ValueError(f"Invalid norm type {norm_type}. Supported types are LayerNorm and TELayerNorm.")
                layers.append(get_layer_norm_class()(output_dim))
            self.model = nn.Sequential(*layers)
        else:
            self.model = nn.Identity()
        if recompute_activation and not isinstance(activation_fn, nn.SiLU):
            raise ValueError(activation_fn)
        self.recompute_activation = recompute_activation

    def forward(self, x, post: Optional[Tensor] = None) -> Tensor:
        """``x``: tensor or tuple of column blocks; ``post`` is added to the result (block residual)."""
        first = x[0] if isinstance(x, (tuple, list)) else x
        if isinstance(self.model, nn.Sequential) and ops.fused_path_enabled(first):
            y = _chain(self.model, x, post)
            if y is not None:
                return y
        if isinstance(x, (tuple, list)):
            x = torch.cat(list(x), dim=-1)
        y = self.model(x)
        return y if post is None else y + post


class MeshGraphEdgeMLPConcat(MeshGraphMLP):
    """Edge MLP on ``cat(efeat, src_feat[src], dst_feat[dst])``."""

    def __init__(self, efeat_dim: int = 512, src_dim: int = 512, dst_dim: int = 512, output_dim: int = 512,
                 hidden_dim: int = 512, hidden_layers: int = 2, activation_fn: nn.Module = nn.SiLU(),
                 norm_type: str = "LayerNorm", bias: bool = True, recompute_activation: bool = False):
        super().__init__(efeat_dim + src_dim + dst_dim, output_dim, hidden_dim, hidden_layers, activation_fn,
                         norm_type, recompute_activation)

    def forward(self, efeat: Tensor, nfeat, graph, post: Optional[Tensor] = None) -> Tensor:
        if ops.fused_path_enabled(efeat) and efeat.dtype == torch.bfloat16:
            gs, gd = gather_src_dst(nfeat, graph)
            return super().forward((efeat, gs, gd), post=post)
        return super().forward(concat_efeat(efeat, nfeat, graph), post=post)


class MeshGraphHeteroEdgeMLPConcat(nn.Module):
    """Two edge MLPs (mesh edges / world edges) over one concatenated edge set."""

    def __init__(self, efeat_dim: int = 512, src_dim: int = 512, dst_dim: int = 512, output_dim: int = 512,
                 hidden_dim: int = 512, hidden_layers: int = 2, activation_fn: nn.Module = nn.SiLU(),
                 norm_type: str = "LayerNorm", bias: bool = True, recompute_activation: bool = False):
        super().__init__()
        cat_dim = efeat_dim + src_dim + dst_dim
        kw = dict(input_dim=cat_dim, output_dim=output_dim, hidden_dim=hidden_dim, hidden_layers=hidden_layers,
                  activation_fn=activation_fn, norm_type=norm_type, recompute_activation=recompute_activation)
        self.mesh_mlp = MeshGraphMLP(**kw)
        self.world_mlp = MeshGraphMLP(**kw)

    def forward(self, mesh_efeat: Tensor, world_efeat: Tensor, nfeat, graph):
        efeat = concat_efeat_hetero(mesh_efeat, world_efeat, nfeat, graph)
        n = len(mesh_efeat)
        return self.mesh_mlp(efeat[0:n]), self.world_mlp(efeat[n:])


class MeshGraphEdgeMLPSum(nn.Module):
    """Edge MLP with the first linear layer split per input ("concat trick"):
    ``efeat W_e^T + (src W_s^T)[src] + (dst W_d^T + b)[dst]``, cheaper when nodes ≪ edges."""

    def __init__(self, efeat_dim: int, src_dim: int, dst_dim: int, output_dim: int = 512, hidden_dim: int = 512,
                 hidden_layers: int = 1, activation_fn: nn.Module = nn.SiLU(), norm_type: str = "LayerNorm",
                 bias: bool = True, recompute_activation: bool = False):
        super().__init__()
        self.efeat_dim, self.src_dim, self.dst_dim = efeat_dim, src_dim, dst_dim
        tmp = nn.Linear(efeat_dim + src_dim + dst_dim, hidden_dim, bias=bias)
        w_e, w_s, w_d = torch.split(tmp.weight, [efeat_dim, src_dim, dst_dim], dim=1)
        self.lin_efeat, self.lin_src, self.lin_dst = nn.Parameter(w_e), nn.Parameter(w_s), nn.Parameter(w_d)
        self.bias = tmp.bias if bias else None
        layers = [activation_fn]
        self.hidden_layers = hidden_layers
        for _ in range(hidden_layers - 1):
            layers += [nn.Linear(hidden_dim, hidden_dim), activation_fn]
        layers.append(nn.Linear(hidden_dim, output_dim))
        self.norm_type = norm_type
        if norm_type is not None:
            if norm_type not in ("LayerNorm", "TELayerNorm"):
                raise ValueError(f"Invalid norm type {norm_type}. Supported types are LayerNorm and TELayerNorm.")
            layers.append(get_layer_norm_class()(output_dim))
        self.model = nn.Sequential(*layers)
        if recompute_activation and not isinstance(activation_fn, nn.SiLU):
            raise ValueError(activation_fn)
        self.recompute_activation = recompute_activation

    def forward_truncated_sum(self, efeat: Tensor, nfeat, graph) -> Tensor:
        src_feat, dst_feat = nfeat if isinstance(nfeat, (tuple, list)) else (nfeat, nfeat)
        mlp_efeat = ops.linear(efeat, self.lin_efeat, None)
        mlp_src = ops.linear(src_feat, self.lin_src, None)
        mlp_dst = ops.linear(dst_feat, self.lin_dst, self.bias)
        return sum_efeat(mlp_efeat, (mlp_src, mlp_dst), graph)

    def forward(self, efeat: Tensor, nfeat, graph, post: Optional[Tensor] = None) -> Tensor:
        y = self.model(self.forward_truncated_sum(efeat, nfeat, graph))
        return y if post is None else y + post
