"""Learned Green's-function-like kernels: one kernel, its tree-accelerated form, and the multiscale sum.

Parity: ``physicsnemo/experimental/models/globe/field_kernel.py`` — ``Kernel`` (``:122``),
``BarnesHutKernel`` (``:745``), ``MultiscaleKernel`` (``:1510``).  Data layout differs from the
reference: instead of nested tensor dictionaries every group of fields is a plain ``dict`` with
dotted names (``"latent.vectors.3"``), and the per-interaction features are assembled directly as
one ``(pairs, features)`` matrix in this order (the order the reference reaches by sorting its
dictionary keys as strings): global scalars, source scalars, log-magnitudes of the global vectors,
of ``r`` and of the source vectors, then one block per Legendre degree with one column per vector
pair.  Names inside a group are sorted.

The tree-accelerated kernel uses the flat near / far lists of
:class:`physicsnemo_b200.mesh.cluster_tree.ClusterTree`: all near pairs and all far (target, node)
pairs go through the same network in chunks and are summed into one packed ``(targets, features)``
buffer with ``index_add_``.
"""
from __future__ import annotations

import itertools
from math import comb
from typing import Dict, Literal, Mapping, Optional, Sequence

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from ....core.module import Module
from ....mesh.cluster_tree import ClusterTree, InteractionPlan, NodeAggregates
from ....mesh.fields import flatten_rank_spec
from ....nn.functional.equivariant_ops import legendre_polynomials, polar_and_dipole_basis, smooth_log, spherical_basis
from ....nn.module.mlp_layers import Mlp
from ....nn.module.pade import Pade

FieldDict = Dict[str, torch.Tensor]


def _names_by_rank(spec: Optional[Mapping]) -> tuple[list[str], list[str]]:
    flat = flatten_rank_spec(spec or {})
    bad = {k: r for k, r in flat.items() if r not in (0, 1)}
    if bad:
        raise ValueError(f"only rank-0 and rank-1 fields are supported, got {bad}")
    return sorted(k for k, r in flat.items() if r == 0), sorted(k for k, r in flat.items() if r == 1)


def flatten_fields(data: Optional[Mapping], prefix: str = "") -> FieldDict:
    """Nested mapping of tensors → flat dict with dotted names."""
    out: FieldDict = {}
    for k, v in dict(data or {}).items():
        name = f"{prefix}.{k}" if prefix else str(k)
        if isinstance(v, Mapping):
            out.update(flatten_fields(v, name))
        else:
            out[name] = v
    return out


def _stack(data: FieldDict, names: Sequence[str], lead: tuple, tail: tuple, like: torch.Tensor) -> torch.Tensor:
    """``(*lead, *tail, len(names))`` tensor of the named fields (an empty last axis when there are none)."""
    if not names:
        return like.new_zeros(lead + tail + (0,))
    return torch.stack([data[n].to(like.dtype) for n in names], dim=-1)


class Kernel(Module):
    r"""One learned kernel ``K(target, source)`` summed over sources with per-source strengths.

    Inputs are made invariant before they reach the network: the displacement
    ``r = (x_t - x_s) / reference_length``, the per-source and the global vectors enter only through
    smoothed log-magnitudes and through Legendre polynomials of the angles between every pair of
    them, scalars enter as they are.  The network output is damped by ``(1 - e^{-|r|^2}) /
    (1 + |r|^2)^{(d-1)/2}`` (regular at the source, decaying like a ``d``-dimensional potential far
    away); vector outputs are linear combinations of a local frame built from ``r`` and the input
    vectors, which keeps them rotation- and parity-equivariant.

    ``output_field_ranks``, ``source_data_ranks`` and ``global_data_ranks`` are (possibly nested)
    mappings ``name → 0 | 1``.  ``forward`` returns ``{name: (n_targets,) or (n_targets, d)}``.
    """

    def __init__(self, *, n_spatial_dims: int, output_field_ranks: Mapping, source_data_ranks: Optional[Mapping] = None,
                 global_data_ranks: Optional[Mapping] = None, smoothing_radius: float = 1e-8,
                 hidden_layer_sizes: Optional[Sequence[int]] = None, n_spherical_harmonics: int = 4,
                 network_type: Literal["pade", "mlp"] = "pade", spectral_norm: bool = False,
                 use_gradient_checkpointing: bool = True, self_regularization_beta: Optional[float] = None):
        super().__init__()
        if n_spatial_dims not in (2, 3):
            raise NotImplementedError(f"{type(self).__name__} supports 2 or 3 spatial dimensions, got {n_spatial_dims}")
        self.n_spatial_dims = n_spatial_dims
        self.output_field_ranks = dict(output_field_ranks)
        self.source_data_ranks = dict(source_data_ranks or {})
        self.global_data_ranks = dict(global_data_ranks or {})
        self.smoothing_radius = smoothing_radius
        self.hidden_layer_sizes = list(hidden_layer_sizes) if hidden_layer_sizes is not None else [64]
        self.n_spherical_harmonics = n_spherical_harmonics
        self.use_gradient_checkpointing = use_gradient_checkpointing
        self._src_scalars, self._src_vectors = _names_by_rank(self.source_data_ranks)
        self._glb_scalars, self._glb_vectors = _names_by_rank(self.global_data_ranks)
        self._out_scalars, self._out_vectors = _names_by_rank(self.output_field_ranks)
        self._out_names = sorted(self._out_scalars + self._out_vectors)
        n_vec = self.n_vectors_in
        self._pairs = list(itertools.combinations(range(n_vec), 2))     # over (global…, source…, r)
        n_g = len(self._glb_vectors)
        self._logmag_order = list(range(n_g)) + [n_vec - 1] + list(range(n_g, n_vec - 1))   # global…, r, source…
        if network_type == "pade":
            self.network = Pade(in_features=self.network_in_features, hidden_features=self.hidden_layer_sizes,
                                out_features=self.network_out_features, spectral_norm=spectral_norm,
                                numerator_order=2, denominator_order=2, use_separate_mlps=False,
                                share_denominator_across_channels=False,
                                self_regularization_beta=self_regularization_beta)
        elif network_type == "mlp":
            self.network = nn.Sequential(
                Mlp(in_features=self.network_in_features, hidden_features=self.hidden_layer_sizes,
                    out_features=self.network_out_features, spectral_norm=spectral_norm, act_layer=nn.SiLU(),
                    final_dropout=False),
                nn.Tanh())
        else:
            raise ValueError(f"Invalid network type: {network_type=!r}; must be one of ['pade', 'mlp']")

    # ------------------------------------------------------------ bookkeeping
    @property
    def n_vectors_in(self) -> int:
        return 1 + len(self._src_vectors) + len(self._glb_vectors)

    @property
    def network_in_features(self) -> int:
        n_vec = self.n_vectors_in
        return len(self._src_scalars) + len(self._glb_scalars) + n_vec + comb(n_vec, 2) * self.n_spherical_harmonics

    @property
    def coeffs_per_vector(self) -> int:
        return 1 + 2 * (self.n_vectors_in - 1)

    @property
    def network_out_features(self) -> int:
        return len(self._out_scalars) + len(self._out_vectors) * self.coeffs_per_vector

    @property
    def packed_width(self) -> int:
        return len(self._out_scalars) + len(self._out_vectors) * self.n_spatial_dims

    @property
    def floats_per_interaction(self) -> int:
        """Rough count of floats alive per (target, source) pair, used to size evaluation chunks."""
        n_vec, d = self.n_vectors_in, self.n_spatial_dims
        return (d * (1 + 2 * n_vec) + 3 * n_vec + len(self._pairs) * (1 + 2 * self.n_spherical_harmonics)
                + 2 * self.network_in_features + sum(self.hidden_layer_sizes) + 2 * self.network_out_features
                + 1 + d * max(1, 2 * n_vec - 1))

    def _check_inputs(self, source_data: FieldDict, global_data: FieldDict) -> None:
        for label, have, want in (("source", source_data, self._src_scalars + self._src_vectors),
                                  ("global", global_data, self._glb_scalars + self._glb_vectors)):
            missing = [n for n in want if n not in have]
            if missing:
                raise ValueError(f"This kernel was instantiated to expect {label} fields {want},\n"
                                 f"but the forward-method input lacks {missing}.")

    def unpack(self, packed: torch.Tensor) -> FieldDict:
        """Split a ``(n, packed_width)`` buffer into named scalar ``(n,)`` and vector ``(n, d)`` fields."""
        out, at = {}, 0
        for name in self._out_names:
            if name in self._out_scalars:
                out[name] = packed[:, at]
                at += 1
            else:
                out[name] = packed[:, at:at + self.n_spatial_dims]
                at += self.n_spatial_dims
        return out

    # ------------------------------------------------------------------ core
    def evaluate_pairs(self, r: torch.Tensor, src_scalars: torch.Tensor, src_vectors: torch.Tensor,
                       glb_scalars: torch.Tensor, glb_vectors: torch.Tensor) -> torch.Tensor:
        """Kernel values of ``P`` interactions, not yet weighted by the source strengths.

        ``r`` ``(P, d)`` is the dimensionless displacement, ``src_scalars`` ``(P, n_ss)``,
        ``src_vectors`` ``(P, d, n_sv)``, ``glb_scalars`` ``(n_gs,)``, ``glb_vectors`` ``(d, n_gv)``.
        Returns the packed fields ``(P, packed_width)``.
        """
        P, d = r.shape
        if torch.is_autocast_enabled(r.device.type):
            dt = torch.get_autocast_dtype(r.device.type)
            r, src_scalars, src_vectors = r.to(dt), src_scalars.to(dt), src_vectors.to(dt)
            glb_scalars, glb_vectors = glb_scalars.to(dt), glb_vectors.to(dt)
        vec = torch.cat([glb_vectors.expand(P, d, -1), src_vectors, r.unsqueeze(-1)], dim=-1)   # (P, d, n_vec)
        mag_sq = (vec * vec).sum(1) + self.smoothing_radius ** 2
        mag = mag_sq.sqrt()
        hat = vec / mag.unsqueeze(1)
        log_mag = smooth_log(mag)
        feats = [glb_scalars.expand(P, -1), src_scalars, log_mag[:, self._logmag_order]]
        if self._pairs:
            k1, k2 = (list(k) for k in zip(*self._pairs))
            cos = (hat[:, :, k1] * hat[:, :, k2]).sum(1)
            scale = smooth_log(mag[:, k1] * mag[:, k2])
            feats += [scale * p for p in legendre_polynomials(cos, self.n_spherical_harmonics + 1)[1:]]
        x = torch.cat(feats, dim=-1)
        if x.shape[-1] != self.network_in_features:
            raise RuntimeError(f"assembled {x.shape[-1]} features, the network expects {self.network_in_features}")
        out = self.network(x)
        r_sq = mag_sq[:, -1:]
        out = out * (-torch.expm1(-r_sq))
        out = out / ((r_sq + 1).sqrt() if d == 2 else (r_sq + 1))
        if not self._out_vectors:
            return out
        r_hat = hat[:, :, -1]
        frame = [r_hat]
        for k in range(vec.shape[-1] - 1):                      # global vectors, then source vectors
            s = log_mag[:, k:k + 1]
            if d == 2:
                e = polar_and_dipole_basis(r_hat=r_hat, n_hat=hat[:, :, k], normalize_basis_vectors=False)[2]
            else:
                e = spherical_basis(r_hat=r_hat, n_hat=hat[:, :, k], normalize_basis_vectors=False)[1]
            frame += [s * hat[:, :, k], s * e]
        basis = torch.stack(frame, dim=-1)                      # (P, d, coeffs_per_vector)
        cols, at, c = [], 0, self.coeffs_per_vector
        for name in self._out_names:
            if name in self._out_scalars:
                cols.append(out[:, at:at + 1])
                at += 1
            else:
                cols.append((basis * out[:, None, at:at + c]).sum(-1))
                at += c
        return torch.cat(cols, dim=-1)

    def _split_inputs(self, source_data, global_data, n_sources: int, like: torch.Tensor):
        source_data, global_data = flatten_fields(source_data), flatten_fields(global_data)
        self._check_inputs(source_data, global_data)
        d = self.n_spatial_dims
        return (_stack(source_data, self._src_scalars, (n_sources,), (), like),
                _stack(source_data, self._src_vectors, (n_sources,), (d,), like),
                _stack(global_data, self._glb_scalars, (), (), like),
                _stack(global_data, self._glb_vectors, (), (d,), like))

    def _check_points(self, source_points, target_points):
        for label, p in (("source_points", source_points), ("target_points", target_points)):
            if p.ndim != 2:
                raise ValueError(f"Expected {label} to be 2-dimensional, got {p.ndim}D tensor with shape {p.shape}")
            if p.shape[-1] != self.n_spatial_dims:
                raise ValueError(f"Expected {label} last dimension to be {self.n_spatial_dims}, got {p.shape[-1]}")

    def forward(self, *, reference_length: torch.Tensor, source_points: torch.Tensor, target_points: torch.Tensor,
                source_strengths: Optional[torch.Tensor] = None, source_data: Optional[Mapping] = None,
                global_data: Optional[Mapping] = None, target_chunk_size: Optional[int] = None) -> FieldDict:
        """Exact all-pairs evaluation: ``out[t] = Σ_s strength[s] · K(x_t, x_s)``."""
        self._check_points(source_points, target_points)
        n_s, n_t = source_points.shape[0], target_points.shape[0]
        if source_strengths is None:
            source_strengths = source_points.new_ones(n_s)
        s_sc, s_vec, g_sc, g_vec = self._split_inputs(source_data, global_data, n_s, source_points)
        step = target_chunk_size or max(n_t, 1)
        pieces = []
        for lo in range(0, n_t, step):
            tp = target_points[lo:lo + step]
            m = tp.shape[0]
            r = ((tp[:, None, :] - source_points[None, :, :]) / reference_length).reshape(m * n_s, -1)
            vals = self.evaluate_pairs(r, s_sc.repeat(m, 1), s_vec.repeat(m, 1, 1), g_sc, g_vec)
            pieces.append(torch.einsum("tsf,s->tf", vals.reshape(m, n_s, -1), source_strengths.to(vals.dtype)))
        packed = torch.cat(pieces) if pieces else source_points.new_zeros(0, self.packed_width)
        return self.unpack(packed)


def _chunk_budget_bytes(device: torch.device) -> int:
    """Memory one evaluation chunk may use: an eighth of the device, 1 GiB on the host."""
    if device.type == "cuda":
        return torch.cuda.get_device_properties(device).total_memory // 8
    return 1 << 30


class BarnesHutKernel(Kernel):
    r"""Tree-accelerated :class:`Kernel`: near pairs exactly, distant source clusters as one virtual source.

    A far cluster is represented by its area-weighted centroid, its area-weighted mean features and
    the sum of its strengths; the same network evaluates it.  ``theta = 0`` reproduces
    :meth:`Kernel.forward`.  ``cluster_tree``, ``target_tree``, ``plan`` and ``aggregates`` can be
    passed in when several kernels share one geometry.
    """

    def __init__(self, *, leaf_size: int = 1, **kernel_args):
        super().__init__(**kernel_args)
        self.leaf_size = leaf_size

    def auto_chunk_size(self, n_pairs: int, device: torch.device) -> int:
        """Pairs per chunk so that a chunk's intermediates (with an autograd margin of 3×) fit the budget."""
        per_pair = 4 * self.floats_per_interaction * 3
        return int(max(4096, min(max(n_pairs, 1), _chunk_budget_bytes(device) // per_pair)))

    def _gather_eval(self, tgt_ids, src_ids, tgt_pts, src_pts, s_sc, s_vec, g_sc, g_vec, reference_length, weights):
        r = (tgt_pts[tgt_ids] - src_pts[src_ids]) / reference_length
        vals = self.evaluate_pairs(r, s_sc[src_ids], s_vec[src_ids], g_sc, g_vec)
        return vals * weights[src_ids].to(vals.dtype).unsqueeze(-1)

    def _accumulate(self, buf, tgt_ids, src_ids, chunk, *args):
        for lo in range(0, tgt_ids.numel(), chunk):
            t, s = tgt_ids[lo:lo + chunk], src_ids[lo:lo + chunk]
            if self.use_gradient_checkpointing and self.training and torch.is_grad_enabled():
                # only the index tensors are saved; the gathered features are rebuilt in backward
                vals = checkpoint(self._gather_eval, t, s, *args, use_reentrant=False)
            else:
                vals = self._gather_eval(t, s, *args)
            buf = buf.index_add(0, t, vals.to(buf.dtype))
        return buf

    def forward(self, *, reference_length: torch.Tensor, source_points: torch.Tensor, target_points: torch.Tensor,
                source_strengths: Optional[torch.Tensor] = None, source_data: Optional[Mapping] = None,
                global_data: Optional[Mapping] = None, theta: float = 1.0, cluster_tree: Optional[ClusterTree] = None,
                target_tree: Optional[ClusterTree] = None, plan: Optional[InteractionPlan] = None,
                source_areas: Optional[torch.Tensor] = None, aggregates: Optional[NodeAggregates] = None,
                chunk_size: Optional[int] = None) -> FieldDict:
        self._check_points(source_points, target_points)
        n_s, n_t = source_points.shape[0], target_points.shape[0]
        dev = source_points.device
        if source_strengths is None:
            source_strengths = source_points.new_ones(n_s)
        if source_areas is None:
            source_areas = source_points.new_ones(n_s)
        source_data = flatten_fields(source_data)
        if plan is None:
            if cluster_tree is None:
                cluster_tree = ClusterTree.from_points(source_points, self.leaf_size)
            if target_tree is None:
                target_tree = (cluster_tree if target_points is source_points
                               else ClusterTree.from_points(target_points, self.leaf_size))
            plan = cluster_tree.find_interactions(target_tree, theta)
        s_sc, s_vec, g_sc, g_vec = self._split_inputs(source_data, global_data, n_s, source_points)
        out_dtype = torch.promote_types(
            torch.get_autocast_dtype(dev.type) if torch.is_autocast_enabled(dev.type) else source_points.dtype,
            source_strengths.dtype)
        buf = torch.zeros(n_t, self.packed_width, dtype=out_dtype, device=dev)
        chunk = chunk_size or self.auto_chunk_size(plan.n_near + plan.n_far, dev)
        if plan.n_near:
            buf = self._accumulate(buf, plan.near_targets, plan.near_sources, chunk, target_points, source_points,
                                   s_sc, s_vec, g_sc, g_vec, reference_length, source_strengths)
        if plan.n_far:
            if cluster_tree is None:
                raise ValueError("a plan with far pairs needs the cluster tree it was made from")
            if aggregates is None:
                wanted = {k: source_data[k] for k in self._src_scalars + self._src_vectors}
                aggregates = cluster_tree.aggregates(source_points, source_areas, wanted)
            n_sc, n_vec, _, _ = self._split_inputs(aggregates.data, global_data, cluster_tree.n_nodes, source_points)
            node_strength = cluster_tree.node_sums(source_strengths)
            buf = self._accumulate(buf, plan.far_targets, plan.far_nodes, chunk, target_points, aggregates.centroid,
                                   n_sc, n_vec, g_sc, g_vec, reference_length, node_strength)
        return self.unpack(buf)


class MultiscaleKernel(Module):
    r"""Sum of independent :class:`BarnesHutKernel` branches, one per named reference length.

    Each branch divides displacements by ``reference_lengths[name] · exp(log_scalefactors[name])``
    (the factor is learned), has its own network and its own per-source strengths.  The logarithms of
    all pairwise reference-length ratios are added to the global scalars
    (``"log_reference_length_ratios.<a>_<b>"``), so a uniform rescaling of the problem leaves the
    features unchanged.  Tree, interaction plan and node aggregates are built once and shared.
    """

    def __init__(self, *, n_spatial_dims: int, output_field_ranks: Mapping, reference_length_names: Sequence[str],
                 source_data_ranks: Optional[Mapping] = None, global_data_ranks: Optional[Mapping] = None,
                 smoothing_radius: float = 1e-8, hidden_layer_sizes: Optional[Sequence[int]] = None,
                 n_spherical_harmonics: int = 4, network_type: Literal["pade", "mlp"] = "pade",
                 spectral_norm: bool = False, use_gradient_checkpointing: bool = True, leaf_size: int = 1,
                 self_regularization_beta: Optional[float] = None):
        super().__init__()
        self.n_spatial_dims = n_spatial_dims
        self.output_field_ranks = dict(output_field_ranks)
        self.reference_length_names = list(reference_length_names)
        self.source_data_ranks = dict(source_data_ranks or {})
        self.global_data_ranks = dict(global_data_ranks or {})
        self.leaf_size = leaf_size
        self._ratio_names = list(itertools.combinations(self.reference_length_names, 2))
        augmented = {**self.global_data_ranks,
                     "log_reference_length_ratios": {f"{a}_{b}": 0 for a, b in self._ratio_names}}
        self.kernels = nn.ModuleDict({
            name: BarnesHutKernel(
                n_spatial_dims=n_spatial_dims, output_field_ranks=output_field_ranks,
                source_data_ranks=source_data_ranks, global_data_ranks=augmented, smoothing_radius=smoothing_radius,
                hidden_layer_sizes=hidden_layer_sizes, n_spherical_harmonics=n_spherical_harmonics,
                network_type=network_type, spectral_norm=spectral_norm,
                use_gradient_checkpointing=use_gradient_checkpointing, leaf_size=leaf_size,
                self_regularization_beta=self_regularization_beta)
            for name in self.reference_length_names})
        self.log_scalefactors = nn.ParameterDict(
            {name: nn.Parameter(torch.zeros(1)) for name in self.reference_length_names})

    def forward(self, *, reference_lengths: Mapping[str, torch.Tensor], source_points: torch.Tensor,
                target_points: torch.Tensor, source_strengths: Optional[Mapping[str, torch.Tensor]] = None,
                source_data: Optional[Mapping] = None, global_data: Optional[Mapping] = None, theta: float = 1.0,
                cluster_tree: Optional[ClusterTree] = None, target_tree: Optional[ClusterTree] = None,
                plan: Optional[InteractionPlan] = None, source_areas: Optional[torch.Tensor] = None) -> FieldDict:
        names = self.reference_length_names
        n_s = source_points.shape[0]
        if source_strengths is None:
            source_strengths = {n: source_points.new_ones(n_s) for n in names}
        for label, have in (("reference_lengths", reference_lengths), ("source_strengths", source_strengths)):
            if set(have.keys()) != set(names):
                raise ValueError(f"This kernel was instantiated to expect {set(names)} {label},\n"
                                 f"but the forward-method input gives {set(have.keys())} {label}.")
        if source_areas is None:
            source_areas = source_points.new_ones(n_s)
        source_data = flatten_fields(source_data)
        if plan is None:
            if cluster_tree is None:
                cluster_tree = ClusterTree.from_points(source_points, self.leaf_size)
            if target_tree is None:
                target_tree = (cluster_tree if target_points is source_points
                               else ClusterTree.from_points(target_points, self.leaf_size))
            plan = cluster_tree.find_interactions(target_tree, theta)
        aggregates = None
        if plan.n_far:
            first = self.kernels[names[0]]
            wanted = {k: source_data[k] for k in first._src_scalars + first._src_vectors}
            aggregates = cluster_tree.aggregates(source_points, source_areas, wanted)
        global_data = flatten_fields(global_data)
        for a, b in self._ratio_names:
            ratio = torch.as_tensor(reference_lengths[a] / reference_lengths[b], device=source_points.device)
            global_data[f"log_reference_length_ratios.{a}_{b}"] = ratio.log().reshape(())
        total: Optional[FieldDict] = None
        for name in names:
            length = reference_lengths[name] * torch.exp(self.log_scalefactors[name])
            piece = self.kernels[name](
                reference_length=length, source_points=source_points, target_points=target_points,
                source_strengths=source_strengths[name], source_data=source_data, global_data=global_data,
                theta=theta, cluster_tree=cluster_tree, target_tree=target_tree, plan=plan,
                source_areas=source_areas, aggregates=aggregates)
            total = piece if total is None else {k: total[k] + piece[k] for k in total}
        return total
