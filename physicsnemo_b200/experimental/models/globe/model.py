"""GLOBE: a boundary-element-style neural operator built from learned Green's-function-like kernels.

Parity: ``physicsnemo/experimental/models/globe/model.py`` (``GLOBE`` ``:66``; hyperlayer evaluation
``:574``, communication hyperlayer ``:672``, forward ``:738``).  Boundary faces act as sources of a
multiscale learned kernel.  A stack of *communication hyperlayers* evaluates the kernels from every
boundary onto every boundary (face centroids as targets) and so produces per-face latent scalars,
latent vectors and per-branch source strengths; the last hyperlayer evaluates the requested output
fields at the query points.  Each face contributes in proportion to its area divided by
``reference_area``, which makes the sum a quadrature of a boundary integral and the result
independent of how finely the boundary is meshed.

Fields are plain dicts with dotted names; boundary meshes are :class:`physicsnemo_b200.mesh.Mesh`
objects whose ``cell_data`` holds the per-face physical features.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Literal, Mapping, Optional, Sequence

import torch
from torch import nn

from ....core.meta import ModelMetaData
from ....core.module import Module
from ....mesh.cluster_tree import ClusterTree, InteractionPlan
from ....mesh.fields import flatten_rank_spec
from ....mesh.mesh import Mesh
from .field_kernel import FieldDict, MultiscaleKernel, flatten_fields


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp: bool = True


def _check_fields(data: FieldDict, ranks: Mapping, label: str, n_dims: int) -> None:
    for name, rank in flatten_rank_spec(ranks).items():
        if name not in data:
            raise KeyError(f"{label} lacks the field {name!r} declared in the rank spec; it has {sorted(data)}")
        trailing = data[name].ndim - (0 if label == "`global_data`" else 1)
        if trailing != rank or (rank == 1 and data[name].shape[-1] != n_dims):
            raise ValueError(f"{label}[{name!r}] has shape {tuple(data[name].shape)}, which is not rank {rank} "
                             f"in {n_dims} dimensions")


class GLOBE(Module):
    r"""Green's-function-like operator for boundary-driven elliptic problems.

    Parameters follow the reference: ``n_spatial_dims`` (2 or 3); ``output_field_ranks`` and
    ``global_data_ranks`` (mappings ``name → 0 | 1``, may be nested); ``boundary_source_data_ranks``
    (one rank mapping per boundary-condition type; the face normal is added automatically);
    ``reference_length_names`` (one kernel branch each); ``reference_area``;
    ``n_communication_hyperlayers``, ``n_latent_scalars``, ``n_latent_vectors``; ``theta`` and
    ``leaf_size`` of the treecode; ``latent_compression_scale`` (``C·asinh(x / C)`` applied to the
    latent outputs of every communication layer, on vector magnitudes for vectors);
    ``tree_build_device`` (where trees and interaction lists are made; ``None`` = the input's device).

    ``forward(prediction_points, boundary_meshes, reference_lengths, global_data=None,
    prediction_chunk_size="auto")`` returns a point-cloud :class:`Mesh` whose ``point_data`` holds the
    output fields (scalars ``(n,)``, vectors ``(n, d)``) under their dotted names.
    """

    def __init__(self, n_spatial_dims: int, output_field_ranks: Mapping, boundary_source_data_ranks: Mapping[str, Mapping],
                 reference_length_names: Sequence[str], reference_area: float, global_data_ranks: Optional[Mapping] = None,
                 n_communication_hyperlayers: int = 2, n_latent_scalars: int = 12, n_latent_vectors: int = 6,
                 smoothing_radius: float = 1e-8, hidden_layer_sizes: Optional[Sequence[int]] = None,
                 n_spherical_harmonics: int = 4, theta: float = 1.0, leaf_size: int = 1,
                 network_type: Literal["pade", "mlp"] = "pade", self_regularization_beta: Optional[float] = None,
                 latent_compression_scale: Optional[float] = None, expand_far_targets: bool = False,
                 use_gradient_checkpointing: bool = True, tree_build_device=None):
        hidden_layer_sizes = list(hidden_layer_sizes) if hidden_layer_sizes is not None else [64, 64, 64]
        global_data_ranks = dict(global_data_ranks or {})
        bc_names = list(boundary_source_data_ranks.keys())
        for rank in flatten_rank_spec(output_field_ranks).values():
            if rank not in (0, 1):
                raise ValueError(f"All leaves of output_field_ranks must be 0 (scalar) or 1 (vector), got {rank!r}")
        for bc in bc_names:
            if "." in bc:
                raise ValueError(f"In `boundary_source_data_ranks`, got bc_name={bc!r};\nBC names must not contain `.`.")
        checks = ((smoothing_radius > 0, f"smoothing_radius must be positive, got {smoothing_radius=!r}"),
                  (theta >= 0, f"theta must be non-negative (0 means exact summation), got {theta=!r}"),
                  (leaf_size >= 1, f"leaf_size must be at least 1, got {leaf_size=!r}"),
                  (reference_area > 0, f"reference_area must be positive, got {reference_area=!r}"),
                  (latent_compression_scale is None or latent_compression_scale > 0,
                   "latent_compression_scale must be positive (use None to disable compression), "
                   f"got {latent_compression_scale=!r}"))
        for ok, message in checks:
            if not ok:
                raise ValueError(message)
        super().__init__(meta=MetaData())
        self.n_spatial_dims = n_spatial_dims
        self.output_field_ranks = dict(output_field_ranks)
        self.boundary_condition_names = bc_names
        self.boundary_source_data_ranks = {k: dict(v) for k, v in boundary_source_data_ranks.items()}
        self.reference_length_names = list(reference_length_names)
        self.register_buffer("reference_area", torch.tensor(float(reference_area)))
        self.global_data_ranks = global_data_ranks
        self.n_communication_hyperlayers = n_communication_hyperlayers
        self.n_latent_scalars, self.n_latent_vectors = n_latent_scalars, n_latent_vectors
        self.smoothing_radius, self.theta, self.leaf_size = smoothing_radius, theta, leaf_size
        self.latent_compression_scale = latent_compression_scale
        # the treecode here never approximates the target side, so this switch changes nothing
        self.expand_far_targets = expand_far_targets
        self.tree_build_device = torch.device(tree_build_device) if tree_build_device is not None else None

        latent_ranks = {"scalars": {str(i): 0 for i in range(n_latent_scalars)},
                        "vectors": {str(i): 1 for i in range(n_latent_vectors)}}
        intermediate = {"strengths": {n: 0 for n in self.reference_length_names}, "latent": latent_ranks}
        layers = []
        for i in range(n_communication_hyperlayers + 1):
            last = i == n_communication_hyperlayers
            layers.append(nn.ModuleDict({
                bc: MultiscaleKernel(
                    n_spatial_dims=n_spatial_dims,
                    output_field_ranks=self.output_field_ranks if last else intermediate,
                    reference_length_names=self.reference_length_names,
                    source_data_ranks=self._source_ranks(bc, include_latents=i > 0, latent_ranks=latent_ranks),
                    global_data_ranks=global_data_ranks, smoothing_radius=smoothing_radius,
                    hidden_layer_sizes=hidden_layer_sizes, n_spherical_harmonics=n_spherical_harmonics,
                    leaf_size=leaf_size, network_type=network_type, self_regularization_beta=self_regularization_beta,
                    use_gradient_checkpointing=use_gradient_checkpointing)
                for bc in bc_names}))
        self.kernel_layers = nn.ModuleList(layers)
        # per-field affine calibration; a bias on a vector field would break rotation equivariance
        flat_out = flatten_rank_spec(self.output_field_ranks)
        self._output_field_order = sorted(flat_out)
        self.final_field_transforms = nn.ModuleList(
            [nn.Linear(1, 1, bias=flat_out[name] == 0) for name in self._output_field_order])

    def _source_ranks(self, bc: str, include_latents: bool, latent_ranks: Mapping) -> dict:
        ranks = {"physical": self.boundary_source_data_ranks[bc], "normals": 1}
        if include_latents:
            ranks["latent"] = latent_ranks
        return ranks

    # ----------------------------------------------------------------- plans
    def _tree(self, points: torch.Tensor) -> ClusterTree:
        where = self.tree_build_device or points.device
        return ClusterTree.from_points(points.detach().to(where), self.leaf_size)

    def _plan(self, source_tree: ClusterTree, target_tree: ClusterTree, device) -> InteractionPlan:
        return source_tree.find_interactions(target_tree, self.theta).to(device)

    # ------------------------------------------------------------ hyperlayers
    def _evaluate_hyperlayer(self, layer: int, target_points: torch.Tensor, state: Dict[str, dict],
                             reference_lengths: Mapping[str, torch.Tensor], global_data: FieldDict,
                             trees: Dict[str, ClusterTree], plans: Dict[str, InteractionPlan]) -> FieldDict:
        """Sum over boundary types of their multiscale kernels, evaluated at ``target_points``."""
        total: Optional[FieldDict] = None
        for bc, s in state.items():
            kernel: MultiscaleKernel = self.kernel_layers[layer][bc]
            piece = kernel(
                reference_lengths=reference_lengths, source_points=s["points"], target_points=target_points,
                source_strengths={n: v * s["areas"] for n, v in s["strengths"].items()},
                source_data=s["data"], global_data=global_data, theta=self.theta,
                cluster_tree=trees[bc], plan=plans[bc], source_areas=s["areas"])
            total = piece if total is None else {k: total[k] + piece[k] for k in total}
        return total

    def _compress(self, t: torch.Tensor) -> torch.Tensor:
        c = self.latent_compression_scale
        if t.ndim == 1:
            return c * torch.arcsinh(t / c)
        r = (t.pow(2).sum(-1, keepdim=True) + self.smoothing_radius ** 2).sqrt()
        return t * (c * torch.arcsinh(r / c) / r)

    def _communicate(self, layer: int, state, reference_lengths, global_data, trees, comm_plans) -> Dict[str, dict]:
        """One boundary-to-boundary layer: every face receives new strengths and latent features."""
        new_state = {}
        for bc, s in state.items():
            out = self._evaluate_hyperlayer(layer, s["points"], state, reference_lengths, global_data, trees,
                                            comm_plans[bc])
            if self.latent_compression_scale is not None:
                out = {k: self._compress(v) for k, v in out.items()}
            data = {k: v for k, v in s["data"].items() if not k.startswith("latent.")}
            data.update({k: v for k, v in out.items() if k.startswith("latent.")})
            strengths = {n: out[f"strengths.{n}"] for n in self.reference_length_names}
            new_state[bc] = dict(s, data=data, strengths=strengths)
        return new_state

    # ---------------------------------------------------------------- forward
    def _validate(self, prediction_points, boundary_meshes, reference_lengths) -> None:
        if prediction_points.ndim != 2:
            raise ValueError(f"Expected 2D prediction_points (N, D), got {prediction_points.ndim}D tensor with "
                             f"shape {tuple(prediction_points.shape)}")
        if prediction_points.shape[-1] != self.n_spatial_dims:
            raise ValueError(f"Expected prediction_points with {self.n_spatial_dims} spatial dims, "
                             f"got {prediction_points.shape[-1]}")
        if set(reference_lengths.keys()) != set(self.reference_length_names):
            raise ValueError(f"This model was instantiated to expect reference lengths "
                             f"{set(self.reference_length_names)!r},\nbut the forward-method input gives "
                             f"{set(reference_lengths.keys())!r}.")
        extra = set(boundary_meshes.keys()) - set(self.boundary_condition_names)
        if extra:
            raise ValueError(f"The input gives boundary meshes of the types {sorted(boundary_meshes)!r},\n"
                             f"but the model was instantiated for {self.boundary_condition_names!r} only.")
        for bc, mesh in boundary_meshes.items():
            if mesh.n_spatial_dims != self.n_spatial_dims:
                raise ValueError(f"Boundary mesh for BC type {bc!r} has {mesh.n_spatial_dims} spatial dims, "
                                 f"but the model expects {self.n_spatial_dims}")

    def forward(self, prediction_points: torch.Tensor, boundary_meshes: Mapping[str, Mesh],
                reference_lengths: Mapping[str, torch.Tensor], global_data: Optional[Mapping] = None,
                prediction_chunk_size: int | Literal["auto"] | None = "auto") -> Mesh:
        self._validate(prediction_points, boundary_meshes, reference_lengths)
        device = prediction_points.device
        wanted_global = flatten_rank_spec(self.global_data_ranks)
        global_all = flatten_fields(global_data)
        _check_fields(global_all, self.global_data_ranks, "`global_data`", self.n_spatial_dims)
        global_data = {k: torch.as_tensor(global_all[k], device=device) for k in wanted_global}

        state: Dict[str, dict] = {}
        for bc, mesh in boundary_meshes.items():
            cell_data = flatten_fields(mesh.cell_data)
            ranks = self.boundary_source_data_ranks[bc]
            _check_fields(cell_data, ranks, f"`boundary_meshes[{bc!r}].cell_data`", self.n_spatial_dims)
            data = {f"physical.{k}": cell_data[k] for k in flatten_rank_spec(ranks)}
            data["normals"] = mesh.cell_normals
            ones = torch.ones(mesh.n_cells, device=device, dtype=mesh.points.dtype)
            state[bc] = dict(points=mesh.cell_centroids, areas=mesh.cell_areas / self.reference_area, data=data,
                             strengths={n: ones for n in self.reference_length_names})

        build_trees = {bc: self._tree(s["points"]) for bc, s in state.items()}
        comm_plans = {tgt: {src: self._plan(build_trees[src], build_trees[tgt], device) for src in state}
                      for tgt in state} if self.n_communication_hyperlayers else {}
        trees = {bc: t.to(device) for bc, t in build_trees.items()}
        for i in range(self.n_communication_hyperlayers):
            state = self._communicate(i, state, reference_lengths, global_data, trees, comm_plans)
        del comm_plans

        n_points = prediction_points.shape[0]
        if prediction_chunk_size == "auto":
            prediction_chunk_size = max(1, sum(m.n_cells for m in boundary_meshes.values()))
        elif prediction_chunk_size is None:
            prediction_chunk_size = max(1, n_points)
        elif not (isinstance(prediction_chunk_size, int) and prediction_chunk_size > 0):
            raise ValueError("Expected prediction_chunk_size to be a positive integer or 'auto' or None, "
                             f"got {prediction_chunk_size=!r}.")
        pieces = []
        for lo in range(0, n_points, prediction_chunk_size):
            chunk = prediction_points[lo:lo + prediction_chunk_size]
            target_tree = self._tree(chunk)
            plans = {bc: self._plan(build_trees[bc], target_tree, device) for bc in state}
            pieces.append(self._evaluate_hyperlayer(self.n_communication_hyperlayers, chunk, state,
                                                    reference_lengths, global_data, trees, plans))
        if pieces:
            fields = {k: torch.cat([p[k] for p in pieces]) for k in pieces[0]}
        else:
            flat_out = flatten_rank_spec(self.output_field_ranks)
            fields = {k: prediction_points.new_zeros((0,) + ((self.n_spatial_dims,) if r else ()))
                      for k, r in flat_out.items()}
        for i, name in enumerate(self._output_field_order):
            t = fields[name]
            fields[name] = self.final_field_transforms[i](t.reshape(-1, 1).to(prediction_points.dtype)).reshape(t.shape)
        return Mesh(points=prediction_points, point_data=fields, global_data=global_data)
