"""DoMINO: decomposable multi-scale neural operator for volume and surface fields around a geometry.

Parity: ``physicsnemo/models/domino/`` — ``model.py`` (``DoMINO``), ``geometry_rep.py`` (``GeoConvOut``, ``GeoProcessor``,
``GeometryRep``, ``scale_sdf``), ``encodings.py`` (``LocalGeometryEncoding``, ``MultiGeometryEncoding``), ``mlps.py``
(``AggregationModel``, ``LocalPointConv``) and ``solutions.py`` (``SolutionCalculatorVolume/Surface``, sphere sampling).
Attribute names follow the reference so its checkpoints load.

Pipeline: (1) geometry points are gathered onto a regular grid by ball queries at several radii, encoded per grid node by an
MLP, smoothed by a 3-D U-Net (or conv) processor and concatenated with an SDF-derived encoding; (2) every query point
samples that grid encoding within local radii (ball query of grid nodes around the point); (3) per output variable a
Fourier-feature basis MLP of the point (and of perturbed / neighbouring points) is concatenated with the positional and
geometry encodings and passed through an aggregation MLP; the centre value and the inverse-distance average of the
neighbours are blended half and half.  Ball queries run on the hash-grid radius-search kernel on CUDA.
"""
from __future__ import annotations

import math
from collections import defaultdict
from typing import Any, Sequence

import torch
import torch.nn as nn

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import get_activation
from ...nn.module.ball_query import BQWarp
from ...nn.module.fourier_layers import FourierMLP, fourier_encode
from ...nn.module.mlp_layers import Mlp
from ..unet import UNet
from .config import DEFAULT_MODEL_PARAMS, Config


def scale_sdf(sdf: torch.Tensor, scaling_factor: float = 0.04) -> torch.Tensor:
    """Squash a signed distance into (-1, 1), resolving the near-surface range."""
    return sdf / (scaling_factor + torch.abs(sdf))


class AggregationModel(Mlp):
    def __init__(self, input_features: int, output_features: int, base_layer: int, activation: nn.Module):
        super().__init__(in_features=input_features, hidden_features=[base_layer] * 4, out_features=output_features, act_layer=activation, drop=0.0)


class LocalPointConv(Mlp):
    def __init__(self, input_features: int, base_layer: int, output_features: int, activation: nn.Module):
        super().__init__(in_features=input_features, hidden_features=base_layer, out_features=output_features, act_layer=activation, drop=0.0)


def _processor_unet(cin, cout, h, activation, attention, normalization=None):
    return UNet(in_channels=cin, out_channels=cout, model_depth=3, feature_map_channels=[h, 2 * h, 4 * h], num_conv_blocks=1, kernel_size=3,
                stride=1, conv_activation=activation, padding=1, padding_mode="zeros", pooling_type="MaxPool3d", pool_size=2,
                normalization=normalization if normalization is not None else ("layernorm" if attention else None),
                use_attn_gate=attention, attn_decoder_feature_maps=[4 * h, 2 * h], attn_feature_map_channels=[2 * h, h],
                attn_intermediate_channels=4 * h, gradient_checkpointing=True)


class GeoConvOut(Module):
    """Encode the ``K`` geometry points found around every grid node into ``base_neurons_in`` channels on the grid."""

    def __init__(self, input_features: int, neighbors_in_radius: int, model_parameters: Any, grid_resolution: list[int] | None = None):
        super().__init__(meta=None)
        grid_resolution = [256, 96, 64] if grid_resolution is None else grid_resolution
        self.fourier_features, self.num_modes = model_parameters.fourier_features, model_parameters.num_modes
        width = input_features * neighbors_in_radius * ((1 + 2 * self.num_modes) if self.fourier_features else 1)
        b = model_parameters.base_neurons
        self.mlp = Mlp(in_features=width, hidden_features=[b, b // 2], out_features=model_parameters.base_neurons_in,
                       act_layer=get_activation(model_parameters.activation), drop=0.0)
        self.grid_resolution, self.neighbors_in_radius = grid_resolution, neighbors_in_radius
        self.activation = get_activation(model_parameters.activation)
        if self.fourier_features:
            self.register_buffer("freqs", torch.exp(torch.linspace(0, math.pi, self.num_modes)))

    def forward(self, x, grid, radius: float = 0.025, neighbors_in_radius: int = 10):
        if x.ndim != 4 or x.shape[-1] != 3:
            raise ValueError(f"Expected x of shape (B, N, K, 3), got shape {tuple(x.shape)}")
        nx, ny, nz = self.grid_resolution[:3]
        x = x.reshape(x.shape[0], nx * ny * nz, self.neighbors_in_radius * 3)
        if self.fourier_features:
            x = torch.cat((x, fourier_encode(x, self.freqs)), dim=-1)
        x = torch.tanh(self.mlp(x))
        return x.reshape(x.shape[0], nx, ny, nz, -1).permute(0, 4, 1, 2, 3)


class GeoProcessor(Module):
    """Plain conv encoder-decoder (three max-pool levels with skip concatenations) over the grid encoding."""

    def __init__(self, input_filters: int, output_filters: int, model_parameters: Any):
        super().__init__(meta=None)
        b = model_parameters.base_filters
        conv = lambda i, o: nn.Conv3d(i, o, kernel_size=3, padding="same")  # noqa: E731
        self.conv1, self.conv2, self.conv3, self.conv3_1 = conv(input_filters, b), conv(b, 2 * b), conv(2 * b, 4 * b), conv(4 * b, 4 * b)
        self.conv4, self.conv5, self.conv6 = conv(4 * b, 2 * b), conv(4 * b, b), conv(2 * b, input_filters)
        self.conv7, self.conv8 = conv(2 * input_filters, input_filters), conv(input_filters, output_filters)
        self.avg_pool, self.max_pool = nn.AvgPool3d((2, 2, 2)), nn.MaxPool3d(2)
        self.upsample = nn.Upsample(scale_factor=2, mode="nearest")
        self.activation = get_activation(model_parameters.activation)

    def forward(self, x):
        if x.ndim != 5:
            raise ValueError(f"Expected x to be 5D (B, C, Nx, Ny, Nz), got {x.ndim}D with shape {tuple(x.shape)}")
        a, pool, up = self.activation, self.max_pool, self.upsample
        x0 = x
        x1 = pool(a(self.conv1(x0)))
        x2 = pool(a(self.conv2(x1)))
        x = a(self.conv3_1(pool(a(self.conv3(x2)))))
        x = torch.cat((up(a(self.conv4(x))), x2), dim=1)
        x = torch.cat((up(a(self.conv5(x))), x1), dim=1)
        x = torch.cat((up(a(self.conv6(x))), x0), dim=1)
        return self.conv8(a(self.conv7(x)))


class GeometryRep(Module):
    """Grid representation of the geometry: one point-cloud channel per radius plus one SDF channel."""

    def __init__(self, input_features: int, radii: Sequence[float], neighbors_in_radius: Sequence[int], hops: int = 1,
                 sdf_scaling_factor: Sequence[float] = (0.04,), model_parameters: Any = None):
        super().__init__(meta=None)
        rep = model_parameters.geometry_rep
        gp, gc = rep.geo_processor, rep.geo_conv
        self.geo_encoding_type = model_parameters.geometry_encoding_type
        self.cross_attention, self.self_attention = gp.cross_attention, gp.self_attention
        self.activation_conv, self.activation_processor = get_activation(gc.activation), gp.activation
        self.sdf_scaling_factor = list(sdf_scaling_factor)
        if gp.processor_type not in ("unet", "conv"):
            raise ValueError(f"Invalid processor_type: {gp.processor_type}. Specify 'unet' or 'conv'.")

        def processor(cin):
            if gp.processor_type == "unet":
                return _processor_unet(cin, gc.base_neurons_out, gp.base_filters, gp.activation, self.self_attention)
            return nn.Sequential(GeoProcessor(input_filters=cin, output_filters=gc.base_neurons_out, model_parameters=gp))

        self.bq_warp = nn.ModuleList([BQWarp(radius=r, neighbors_in_radius=k) for r, k in zip(radii, neighbors_in_radius)])
        self.geo_processors = nn.ModuleList([processor(gc.base_neurons_in) for _ in radii])
        self.geo_conv_out = nn.ModuleList([GeoConvOut(input_features=input_features, neighbors_in_radius=k, model_parameters=gc,
                                                      grid_resolution=model_parameters.interp_res) for k in neighbors_in_radius])
        self.geo_processor_out = nn.ModuleList([nn.Conv3d(gc.base_neurons_out, 1, kernel_size=3, padding="same") for _ in radii])
        self.geo_processor_sdf = processor(5 + len(self.sdf_scaling_factor))
        self.radii, self.neighbors_in_radius, self.hops = radii, neighbors_in_radius, hops
        self.geo_processor_sdf_out = nn.Conv3d(gc.base_neurons_out, 1, kernel_size=3, padding="same")
        if self.cross_attention:
            self.combined_unet = _processor_unet(1 + len(radii), 1 + len(radii), gp.base_filters, gp.activation, True, "layernorm")

    def forward(self, x, p_grid, sdf):
        if x.ndim != 3 or x.shape[-1] != 3:
            raise ValueError(f"Expected x of shape (B, N, 3), got shape {tuple(x.shape)}")
        if p_grid.ndim != 5 or p_grid.shape[-1] != 3:
            raise ValueError(f"Expected p_grid of shape (B, Nx, Ny, Nz, 3), got shape {tuple(p_grid.shape)}")
        if sdf.ndim != 4:
            raise ValueError(f"Expected sdf of shape (B, Nx, Ny, Nz), got {sdf.ndim}D with shape {tuple(sdf.shape)}")
        if self.geo_encoding_type not in ("both", "stl", "sdf"):
            raise ValueError(f"Invalid geo_encoding_type: {self.geo_encoding_type}. Must be 'both', 'stl', or 'sdf'.")
        parts = []
        if self.geo_encoding_type in ("both", "stl"):
            for j in range(len(self.radii)):
                _, k_short = self.bq_warp[j](x, p_grid)
                enc = self.geo_conv_out[j](k_short, p_grid)
                for _ in range(self.hops):
                    enc = enc + self.geo_processors[j](enc) / self.hops
                parts.append(self.geo_processor_out[j](enc))
        if self.geo_encoding_type in ("both", "sdf"):
            s = sdf.unsqueeze(1)
            binary = torch.where(s >= 0, 0.0, 1.0)
            gx, gy, gz = torch.gradient(s, dim=[2, 3, 4])
            scaled = torch.cat([scale_sdf(s, f) for f in self.sdf_scaling_factor], dim=1)
            parts.append(self.geo_processor_sdf_out(self.geo_processor_sdf(torch.cat((s, scaled, binary, gx, gy, gz), 1))))
        encoding_g = torch.cat(parts, dim=1)
        return self.combined_unet(encoding_g) if self.cross_attention else encoding_g


class LocalGeometryEncoding(Module):
    """Sample every channel of the grid encoding at the grid nodes within ``radius`` of each point, then mix by an MLP."""

    def __init__(self, radius: float, neighbors_in_radius: int, total_neighbors_in_radius: int, base_layer: int, activation: nn.Module,
                 grid_resolution: Sequence[int]):
        super().__init__(meta=None)
        self.bq_warp = BQWarp(radius=radius, neighbors_in_radius=neighbors_in_radius)
        self.local_point_conv = LocalPointConv(input_features=total_neighbors_in_radius, base_layer=base_layer,
                                               output_features=neighbors_in_radius, activation=activation)
        self.grid_resolution = grid_resolution

    def forward(self, encoding_g, volume_mesh_centers, p_grid):
        if encoding_g.ndim != 5:
            raise ValueError(f"Expected encoding_g to be 5D (B, C, Nx, Ny, Nz), got {encoding_g.ndim}D with shape {tuple(encoding_g.shape)}")
        if volume_mesh_centers.ndim != 3 or volume_mesh_centers.shape[-1] != 3:
            raise ValueError(f"Expected volume_mesh_centers of shape (B, N, 3), got shape {tuple(volume_mesh_centers.shape)}")
        B, C = encoding_g.shape[:2]
        mapping, _ = self.bq_warp(volume_mesh_centers, p_grid.reshape(B, -1, 3), reverse_mapping=False)
        mapping = mapping.long()                                                    # [B, N, K] grid-node ids, 0 where empty
        mask = mapping != 0
        flat = encoding_g.reshape(B, C, -1)
        idx = mapping.reshape(B, 1, -1).expand(-1, C, -1)
        sampled = torch.gather(flat, 2, idx).reshape(B, C, *mapping.shape[1:]) * mask.unsqueeze(1)   # one gather for all channels
        sampled = sampled.permute(0, 2, 1, 3).reshape(B, mapping.shape[1], -1)      # channel-major neighbour features
        return self.local_point_conv(sampled)


class MultiGeometryEncoding(Module):
    def __init__(self, radii, neighbors_in_radius, geo_encoding_type: str, n_upstream_radii: int, base_layer: int, activation: nn.Module,
                 grid_resolution):
        super().__init__(meta=None)
        self.local_geo_encodings = nn.ModuleList([
            LocalGeometryEncoding(radius=r, neighbors_in_radius=n,
                                  total_neighbors_in_radius=self.calculate_total_neighbors_in_radius(geo_encoding_type, n, n_upstream_radii),
                                  base_layer=base_layer, activation=activation, grid_resolution=grid_resolution)
            for r, n in zip(radii, neighbors_in_radius)])

    @staticmethod
    def calculate_total_neighbors_in_radius(geo_encoding_type: str, neighbors_in_radius: int, n_upstream_radii: int) -> int:
        if geo_encoding_type == "both":
            return neighbors_in_radius * (n_upstream_radii + 1)
        if geo_encoding_type == "stl":
            return neighbors_in_radius * n_upstream_radii
        if geo_encoding_type == "sdf":
            return neighbors_in_radius
        raise ValueError(f"Invalid geo_encoding_type: {geo_encoding_type}. Must be 'both', 'stl', or 'sdf'.")

    def forward(self, encoding_g, volume_mesh_centers, p_grid):
        return torch.cat([enc(encoding_g, volume_mesh_centers, p_grid) for enc in self.local_geo_encodings], dim=-1)


# ---- solution calculators --------------------------------------------------------------------------------------------
def apply_parameter_encoding(mesh_centers, global_params_values, global_params_reference):
    """Global parameters divided by their references, broadcast to every point: ``[B, N, n_params]``."""
    ratio = (global_params_values / global_params_reference).squeeze(-1)
    return ratio.unsqueeze(1).expand(-1, mesh_centers.shape[1], -1)


def sample_sphere(center, r: float, num_points: int):
    c = center.unsqueeze(2).expand(-1, -1, num_points, -1)
    d = torch.randn_like(c)
    d = d / torch.norm(d, dim=-1, keepdim=True)
    return c + d * (r * torch.pow(torch.rand_like(c), 1 / 3))


def sample_sphere_shell(center, r_inner: float, r_outer: float, num_points: int):
    c = center.unsqueeze(2).expand(-1, -1, num_points, -1)
    d = torch.randn_like(c)
    d = d / torch.norm(d, dim=-1, keepdim=True)
    return c + d * torch.pow(torch.rand_like(c) * (r_outer ** 3 - r_inner ** 3) + r_inner ** 3, 1 / 3)


class _SolutionCalculator(Module):
    def __init__(self, num_variables, num_sample_points, encode_parameters, parameter_model, aggregation_model, nn_basis):
        super().__init__(meta=None)
        self.num_variables, self.num_sample_points, self.encode_parameters = num_variables, num_sample_points, encode_parameters
        self.parameter_model, self.aggregation_model, self.nn_basis = parameter_model, aggregation_model, nn_basis
        if encode_parameters and parameter_model is None:
            raise ValueError("Parameter model is required when encode_parameters is True")

    def _features(self, centers, values, reference, encoding_node, encoding_g):
        shared = [encoding_node, encoding_g]
        if self.encode_parameters:
            shared.append(self.parameter_model(apply_parameter_encoding(centers, values, reference)))
        return torch.cat(shared, dim=-1)

    def _blend(self, f: int, points, centre_xyz, shared, keep=None):
        """Centre prediction blended with the inverse-distance mean over the other sample points of ``points [B,N,P,F]``."""
        out_c, num, den = None, None, None
        for p in range(points.shape[2]):
            pt = points[:, :, p]
            val = self.aggregation_model[f](torch.cat((self.nn_basis[f](pt), shared), dim=-1))
            if keep is not None:
                keep.append(val)
            if p == 0:
                out_c = val
                continue
            w = 1.0 / torch.norm(pt[..., :3] - centre_xyz, dim=-1, keepdim=True)
            num = val * w if num is None else num + val * w
            den = w if den is None else den + w
        return 0.5 * out_c + 0.5 * num / den if self.num_sample_points > 1 and num is not None else out_c


class SolutionCalculatorVolume(_SolutionCalculator):
    def __init__(self, num_variables, num_sample_points, noise_intensity, encode_parameters, return_volume_neighbors, parameter_model,
                 aggregation_model, nn_basis):
        super().__init__(num_variables, num_sample_points, encode_parameters, parameter_model, aggregation_model, nn_basis)
        self.noise_intensity, self.return_volume_neighbors = noise_intensity, return_volume_neighbors

    def forward(self, volume_mesh_centers, encoding_g, encoding_node, global_params_values, global_params_reference):
        if volume_mesh_centers.ndim != 3 or volume_mesh_centers.shape[-1] != 3:
            raise ValueError(f"Expected volume_mesh_centers of shape (B, N, 3), got shape {tuple(volume_mesh_centers.shape)}")
        if encoding_g.ndim != 3 or encoding_node.ndim != 3:
            raise ValueError("encoding_g and encoding_node must be 3D (B, N, D)")
        shared = self._features(volume_mesh_centers, global_params_values, global_params_reference, encoding_node, encoding_g)
        r = 1 / self.noise_intensity
        pts, neighbors = [volume_mesh_centers.unsqueeze(2)], None
        hop1 = sample_sphere(volume_mesh_centers, r, self.num_sample_points)
        pts.append(hop1)
        if self.return_volume_neighbors:
            n1 = self.num_sample_points
            n2 = n1 // 2 if n1 != 1 else 1
            neighbors = defaultdict(list)
            neighbors[0] = list(range(1, n1 + 1))
            for i in range(n1):
                pts.append(sample_sphere_shell(hop1[:, :, i], r, 2 * r, n2))
                neighbors[i + 1] = list(range(1 + n1 + i * n2, 1 + n1 + (i + 1) * n2))
            neighbors = dict(neighbors)
        pts = torch.cat(pts, dim=2)
        outs, fields = [], []
        for f in range(self.num_variables):
            keep = [] if self.return_volume_neighbors else None
            outs.append(self._blend(f, pts, volume_mesh_centers, shared, keep))
            if keep is not None:
                fields.append(torch.stack(keep, dim=2))
        out = torch.cat(outs, dim=-1)
        if self.return_volume_neighbors:
            return out, pts, torch.cat(fields, dim=3), neighbors
        return out


class SolutionCalculatorSurface(_SolutionCalculator):
    def __init__(self, num_variables, num_sample_points, encode_parameters, use_surface_normals, use_surface_area, parameter_model,
                 aggregation_model, nn_basis):
        super().__init__(num_variables, num_sample_points, encode_parameters, parameter_model, aggregation_model, nn_basis)
        self.use_surface_normals, self.use_surface_area = use_surface_normals, use_surface_area

    def forward(self, surface_mesh_centers, encoding_g, encoding_node, surface_mesh_neighbors, surface_normals, surface_neighbors_normals,
                surface_areas, surface_neighbors_areas, global_params_values, global_params_reference):
        if surface_mesh_centers.ndim != 3 or surface_mesh_centers.shape[-1] != 3:
            raise ValueError(f"Expected surface_mesh_centers of shape (B, N, 3), got shape {tuple(surface_mesh_centers.shape)}")
        if surface_mesh_neighbors.ndim != 4 or surface_mesh_neighbors.shape[-1] != 3:
            raise ValueError(f"Expected surface_mesh_neighbors of shape (B, N, K, 3), got shape {tuple(surface_mesh_neighbors.shape)}")
        shared = self._features(surface_mesh_centers, global_params_values, global_params_reference, encoding_node, encoding_g)
        centre, neigh = [surface_mesh_centers], [surface_mesh_neighbors]
        many = self.num_sample_points > 1
        if self.use_surface_normals:
            centre.append(surface_normals)
            if many:
                neigh.append(surface_neighbors_normals)
        if self.use_surface_area:
            centre.append(torch.log(surface_areas) / 10)
            if many:
                neigh.append(torch.log(surface_neighbors_areas) / 10)
        centre, neigh = torch.cat(centre, dim=-1), torch.cat(neigh, dim=-1)
        outs = []
        for f in range(self.num_variables):
            out_c, num, den = None, None, None
            for p in range(self.num_sample_points):
                pt = centre if p == 0 else neigh[:, :, p - 1] + 1e-6
                val = self.aggregation_model[f](torch.cat((self.nn_basis[f](pt), shared), dim=-1))
                if p == 0:
                    out_c = val
                    continue
                w = 1.0 / torch.norm(centre - pt, dim=-1, keepdim=True)
                num = val * w if num is None else num + val * w
                den = w if den is None else den + w
            outs.append(0.5 * out_c + 0.5 * num / den if many else out_c)
        return torch.cat(outs, dim=-1)


# ---- the model -------------------------------------------------------------------------------------------------------
class DoMINO(Module):
    """``forward(data_dict) -> (volume_prediction | None, surface_prediction | None)``."""

    def __init__(self, input_features: int, output_features_vol: int | None = None, output_features_surf: int | None = None,
                 global_features: int = 2, model_parameters: Any = None):
        super().__init__(meta=ModelMetaData(name="DoMINO"))
        mp = DEFAULT_MODEL_PARAMS if model_parameters is None else (model_parameters if isinstance(model_parameters, Config) else Config.from_hydra(model_parameters))
        if hasattr(self, "_args"):
            self._args["__args__"]["model_parameters"] = mp
        if output_features_vol is None and output_features_surf is None:
            raise ValueError("At least one of `output_features_vol` or `output_features_surf` must be specified")
        self.output_features_vol = self.num_variables_vol = output_features_vol
        self.output_features_surf = self.num_variables_surf = output_features_surf
        self.num_sample_points_surface, self.num_sample_points_volume = mp.num_neighbors_surface, mp.num_neighbors_volume
        self.combined_vol_surf = mp.combine_volume_surface
        gc, gp = mp.geometry_rep.geo_conv, mp.geometry_rep.geo_processor
        self.activation_processor = gp.activation
        if self.combined_vol_surf:
            cin = 2 + len(gc.volume_radii) + len(gc.surface_radii)
            self.combined_unet_surf = _processor_unet(cin, 1 + len(gc.surface_radii), 8, gp.activation, True, "layernorm")
            self.combined_unet_vol = _processor_unet(cin, 1 + len(gc.volume_radii), 8, gp.activation, True, "layernorm")
        self.global_features = global_features
        mode = getattr(mp, "solution_calculation_mode", "two-loop") if "solution_calculation_mode" in mp else "two-loop"
        if mode not in ("one-loop", "two-loop"):
            raise ValueError(f"Invalid solution_calculation_mode: {mode}, select 'one-loop' or 'two-loop'.")
        self.solution_calculation_mode = mode
        self.grid_resolution = mp.interp_res
        self.use_surface_normals, self.use_surface_area = mp.use_surface_normals, mp.use_surface_area
        self.encode_parameters, self.geo_encoding_type = mp.encode_parameters, mp.geometry_encoding_type
        feats_surf = input_features + ((4 if self.use_surface_area else 3) if self.use_surface_normals else 0)

        def fmlp(cin, section, base):
            return FourierMLP(input_features=cin, fourier_features=section.fourier_features, num_modes=section.num_modes, base_layer=base,
                              activation=get_activation(section.activation))

        base_p = 0
        if self.encode_parameters:
            base_p = mp.parameter_model.base_layer
            self.parameter_model = fmlp(global_features, mp.parameter_model, base_p)
        self.geo_rep_volume = GeometryRep(input_features=input_features, radii=gc.volume_radii, neighbors_in_radius=gc.volume_neighbors_in_radius,
                                          hops=gc.volume_hops, sdf_scaling_factor=gp.volume_sdf_scaling_factor, model_parameters=mp)
        self.geo_rep_surface = GeometryRep(input_features=input_features, radii=gc.surface_radii, neighbors_in_radius=gc.surface_neighbors_in_radius,
                                           hops=gc.surface_hops, sdf_scaling_factor=gp.surface_sdf_scaling_factor, model_parameters=mp)
        base_nn = mp.nn_basis_functions.base_layer
        if output_features_surf is not None:
            self.nn_basis_surf = nn.ModuleList([fmlp(feats_surf, mp.nn_basis_functions, base_nn) for _ in range(output_features_surf)])
        if output_features_vol is not None:
            self.nn_basis_vol = nn.ModuleList([fmlp(input_features, mp.nn_basis_functions, base_nn) for _ in range(output_features_vol)])
        pe = mp.position_encoder
        self.activation = get_activation(mp.activation)
        self.use_sdf_in_basis_func = mp.use_sdf_in_basis_func
        self.sdf_scaling_factor = gp.volume_sdf_scaling_factor
        if output_features_vol is not None:
            self.fc_p_vol = fmlp(7 + len(self.sdf_scaling_factor) if mp.use_sdf_in_basis_func else 3, pe, pe.base_neurons)
        if output_features_surf is not None:
            self.fc_p_surf = fmlp(3, pe, pe.base_neurons)
        gl = mp.geometry_local
        act_local = get_activation(mp.local_point_conv.activation)
        self.surface_local_geo_encodings = MultiGeometryEncoding(radii=gl.surface_radii, neighbors_in_radius=gl.surface_neighbors_in_radius,
                                                                 geo_encoding_type=self.geo_encoding_type, n_upstream_radii=len(gc.surface_radii),
                                                                 base_layer=512, activation=act_local, grid_resolution=self.grid_resolution)
        self.volume_local_geo_encodings = MultiGeometryEncoding(radii=gl.volume_radii, neighbors_in_radius=gl.volume_neighbors_in_radius,
                                                                geo_encoding_type=self.geo_encoding_type, n_upstream_radii=len(gc.volume_radii),
                                                                base_layer=512, activation=act_local, grid_resolution=self.grid_resolution)
        agg = mp.aggregation_model

        def agg_models(n, geo_width):
            return nn.ModuleList([AggregationModel(input_features=pe.base_neurons + base_nn + geo_width + base_p, output_features=1,
                                                   base_layer=agg.base_layer, activation=get_activation(agg.activation)) for _ in range(n)])

        pm = self.parameter_model if self.encode_parameters else None
        if output_features_surf is not None:
            self.agg_model_surf = agg_models(output_features_surf, sum(gl.surface_neighbors_in_radius))
            self.solution_calculator_surf = SolutionCalculatorSurface(
                num_variables=output_features_surf, num_sample_points=self.num_sample_points_surface, use_surface_normals=self.use_surface_normals,
                use_surface_area=self.use_surface_area, encode_parameters=self.encode_parameters, parameter_model=pm,
                aggregation_model=self.agg_model_surf, nn_basis=self.nn_basis_surf)
        if output_features_vol is not None:
            self.agg_model_vol = agg_models(output_features_vol, sum(gl.volume_neighbors_in_radius))
            self.solution_calculator_vol = SolutionCalculatorVolume(
                num_variables=output_features_vol, num_sample_points=self.num_sample_points_volume, noise_intensity=50,
                return_volume_neighbors=bool(mp.get("return_volume_neighbors", False)), encode_parameters=self.encode_parameters,
                parameter_model=pm, aggregation_model=self.agg_model_vol, nn_basis=self.nn_basis_vol)

    @staticmethod
    def _normalise(points, min_max):
        lo, hi = min_max[:, 0].unsqueeze(1), min_max[:, 1].unsqueeze(1)
        return 2.0 * (points - lo) / (hi - lo) - 1

    def forward(self, data_dict: dict):
        need = ["geometry_coordinates", "surf_grid", "sdf_surf_grid", "global_params_values", "global_params_reference"]
        if self.output_features_vol is not None:
            need += ["grid", "sdf_grid", "sdf_nodes", "pos_volume_closest", "pos_volume_center_of_mass", "volume_mesh_centers"]
        if self.output_features_surf is not None:
            need += ["pos_surface_center_of_mass", "surface_mesh_centers", "surface_mesh_neighbors", "surface_normals",
                     "surface_neighbors_normals", "surface_areas", "surface_neighbors_areas"]
        missing = [k for k in need if k not in data_dict]
        if missing:
            raise ValueError(f"Missing required keys in data_dict: {missing}")
        d = data_dict
        geo, values, reference = d["geometry_coordinates"], d["global_params_values"], d["global_params_reference"]
        enc_g_vol = enc_g_surf = None
        if self.output_features_vol is not None:
            geo_v = self._normalise(geo, d["volume_min_max"]) if "volume_min_max" in d else geo
            enc_g_vol = self.geo_rep_volume(geo_v, d["grid"], d["sdf_grid"])
            if self.use_sdf_in_basis_func:
                scaled = torch.cat([scale_sdf(d["sdf_nodes"], f) for f in self.sdf_scaling_factor], dim=-1)
                node = torch.cat((d["sdf_nodes"], scaled, d["pos_volume_closest"], d["pos_volume_center_of_mass"]), dim=-1)
            else:
                node = d["pos_volume_center_of_mass"]
            enc_node_vol = self.fc_p_vol(node)
        if self.output_features_surf is not None:
            geo_s = self._normalise(geo, d["surface_min_max"]) if "surface_min_max" in d else geo
            enc_g_surf = self.geo_rep_surface(geo_s, d["surf_grid"], d["sdf_surf_grid"])
            enc_node_surf = self.fc_p_surf(d["pos_surface_center_of_mass"])
        if enc_g_vol is not None and enc_g_surf is not None and self.combined_vol_surf:
            both = torch.cat((enc_g_vol, enc_g_surf), dim=1)
            enc_g_surf, enc_g_vol = self.combined_unet_surf(both), self.combined_unet_vol(both)
        out_vol = out_surf = None
        if self.output_features_vol is not None:
            local = self.volume_local_geo_encodings(0.5 * enc_g_vol, d["volume_mesh_centers"], d["grid"])
            out_vol = self.solution_calculator_vol(d["volume_mesh_centers"], local, enc_node_vol, values, reference)
        if self.output_features_surf is not None:
            local = self.surface_local_geo_encodings(0.5 * enc_g_surf, d["surface_mesh_centers"], d["surf_grid"])
            out_surf = self.solution_calculator_surf(d["surface_mesh_centers"], local, enc_node_surf, d["surface_mesh_neighbors"],
                                                     d["surface_normals"], d["surface_neighbors_normals"], d["surface_areas"].unsqueeze(-1),
                                                     d["surface_neighbors_areas"].unsqueeze(-1), values, reference)
        return out_vol, out_surf
