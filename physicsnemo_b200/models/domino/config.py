"""Attribute-access configuration of DoMINO and its defaults (parity: ``physicsnemo/models/domino/config.py``)."""
from __future__ import annotations

from dataclasses import fields, is_dataclass
from typing import Any


class Config(dict):
    """``dict`` whose keys read and write as attributes; nested dicts are wrapped on the way in."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        for k, v in list(self.items()):
            if isinstance(v, dict) and not isinstance(v, Config):
                self[k] = Config(v)

    def __getattr__(self, key: str) -> Any:
        try:
            return self[key]
        except KeyError:
            raise AttributeError(f"'{type(self).__name__}' has no attribute '{key}'") from None

    def __setattr__(self, key: str, value: Any):
        self[key] = Config(value) if isinstance(value, dict) and not isinstance(value, Config) else value

    def __delattr__(self, key: str):
        try:
            del self[key]
        except KeyError:
            raise AttributeError(f"'{type(self).__name__}' has no attribute '{key}'") from None

    @classmethod
    def from_hydra(cls, cfg: Any) -> "Config":
        """Accept a mapping, an OmegaConf-like node (anything with ``keys``), a dataclass instance or a plain object."""
        if cfg is None:
            return cls()
        if isinstance(cfg, dict):
            return cls(cfg)
        if is_dataclass(cfg) and not isinstance(cfg, type):
            return cls(_dataclass_to_dict(cfg))
        if hasattr(cfg, "keys") and hasattr(cfg, "__getitem__"):
            return cls(_to_container(cfg))
        if hasattr(cfg, "__dict__"):
            return cls({k: v for k, v in vars(cfg).items() if not k.startswith("_")})
        raise TypeError(f"Cannot convert {type(cfg)} to Config")


def _to_container(node):
    if hasattr(node, "keys") and hasattr(node, "__getitem__"):
        return {k: _to_container(node[k]) for k in node.keys()}
    if not isinstance(node, (str, bytes)) and hasattr(node, "__iter__") and not isinstance(node, (list, tuple)):
        return [_to_container(v) for v in node]
    return node


def _dataclass_to_dict(obj: Any) -> dict:
    out = {}
    for f in fields(obj):
        v = getattr(obj, f.name)
        out[f.name] = _dataclass_to_dict(v) if is_dataclass(v) and not isinstance(v, type) else v
    return out


DEFAULT_MODEL_PARAMS = Config({
    "model_type": "combined", "activation": "gelu", "interp_res": [128, 64, 64], "use_sdf_in_basis_func": True,
    "positional_encoding": False, "surface_neighbors": True, "num_neighbors_surface": 7, "num_neighbors_volume": 10,
    "use_surface_normals": True, "use_surface_area": True, "encode_parameters": False, "combine_volume_surface": False,
    "geometry_encoding_type": "both", "solution_calculation_mode": "two-loop",
    "geometry_rep": {
        "base_filters": 8,
        "geo_conv": {"base_neurons": 32, "base_neurons_in": 1, "base_neurons_out": 1, "surface_hops": 1, "volume_hops": 1,
                     "volume_radii": [0.1, 0.5, 1.0, 2.5], "volume_neighbors_in_radius": [32, 64, 128, 256],
                     "surface_radii": [0.01, 0.05, 1.0], "surface_neighbors_in_radius": [8, 16, 128], "activation": "gelu",
                     "fourier_features": False, "num_modes": 5},
        "geo_processor": {"base_filters": 8, "activation": "gelu", "processor_type": "unet", "self_attention": False,
                          "cross_attention": False, "volume_sdf_scaling_factor": [0.04],
                          "surface_sdf_scaling_factor": [0.01, 0.02, 0.04]},
    },
    "geometry_local": {"base_layer": 512, "volume_neighbors_in_radius": [64, 128], "surface_neighbors_in_radius": [32, 128],
                       "volume_radii": [0.1, 0.25], "surface_radii": [0.05, 0.25]},
    "nn_basis_functions": {"base_layer": 512, "fourier_features": True, "num_modes": 5, "activation": "gelu"},
    "local_point_conv": {"activation": "gelu"},
    "aggregation_model": {"base_layer": 512, "activation": "gelu"},
    "position_encoder": {"base_neurons": 512, "activation": "gelu", "fourier_features": True, "num_modes": 5},
    "parameter_model": {"base_layer": 512, "fourier_features": False, "num_modes": 5, "activation": "gelu"},
})
