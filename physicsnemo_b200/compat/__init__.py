"""Import-path compatibility.

Parity: ``physicsnemo/compat/__init__.py`` — ``install()`` aliases historical module paths (``*.utils.filesystem``,
``*.models.layers.*``, ``*.launch.logging`` …) and moved objects to their current homes, each with a
``DeprecationWarning``.  Additionally ``install(alias_top_level=True)`` registers this package under the name
``physicsnemo`` so that code written against the reference imports runs unchanged.
"""
import importlib
import sys
import types
import warnings

_PKG = "physicsnemo_b200"

COMPAT_MAP = {
    "utils.filesystem": "core.filesystem",
    "utils.version_check": "core.version_check",
    "models.meta": "core.meta",
    "models.module": "core.module",
    "utils.neighbors": "nn.functional",
    "utils.sdf": "nn.functional.geometry.sdf",
    "models.layers": "nn",
    **{f"models.layers.{m}": f"nn.module.{m}" for m in (
        "activations", "attention_layers", "ball_query", "conv_layers", "dgm_layers", "drop", "fourier_layers",
        "fully_connected_layers", "kan_layers", "mlp_layers", "resample_layers", "siren_layers", "spectral_layers",
        "transformer_decoder", "transformer_layers", "weight_fact", "weight_norm")},
    "models.layers.interpolation": "nn.functional.interpolation",
    "utils.diffusion": "diffusion.utils",
    "models.diffusion.corrdiff_utils": "diffusion.samplers",
    "metrics.diffusion": "diffusion.metrics",
    "utils.patching": "diffusion.multi_diffusion.patching",
    "launch.utils.checkpoint": "utils.checkpoint",
    "launch.logging": "utils.logging",
    "distributed.shard_tensor": "parallel.shard_tensor",
}

OBJECT_COMPAT_MAP = {
    "models.diffusion.AttentionOp": "nn.module.attention_layers.AttentionOp",
    "models.diffusion.layers.Attention": "nn.module.attention_layers.UNetAttention",
    "models.diffusion.Conv2D": "nn.module.conv_layers.Conv2d",
    "models.diffusion.FourierEmbedding": "nn.module.embedding_layers.FourierEmbedding",
    "models.diffusion.GroupNorm": "nn.module.group_norm.GroupNorm",
    "models.diffusion.get_group_norm": "nn.module.group_norm.get_group_norm",
    "models.diffusion.Linear": "nn.module.fully_connected_layers.Linear",
    "models.diffusion.PositionalEmbedding": "nn.module.embedding_layers.PositionalEmbedding",
    "models.diffusion.UNetBlock": "nn.module.unet_layers.UNetBlock",
    **{f"models.diffusion.{n}": f"models.diffusion_unets.{n}" for n in (
        "SongUNet", "SongUNetPosEmbd", "SongUNetPosLtEmbd", "DhariwalUNet", "UNet", "StormCastUNet")},
    **{f"models.diffusion.{n}": f"diffusion.preconditioners.{n}" for n in (
        "EDMPrecond", "EDMPrecondSuperResolution", "EDMPrecondSR", "VEPrecond", "VPPrecond", "iDDPMPrecond",
        "VEPrecond_dfsr_cond", "VEPrecond_dfsr")},
}


def _ensure_parents(name: str) -> None:
    parts = name.split(".")
    for i in range(1, len(parts)):
        parent = ".".join(parts[:i])
        if parent in sys.modules:
            continue
        try:
            importlib.import_module(parent)
        except ImportError:
            mod = types.ModuleType(parent)
            mod.__path__ = []  # mark as package so that sub-module aliases resolve
            sys.modules[parent] = mod
            if i > 1:
                setattr(sys.modules[".".join(parts[: i - 1])], parts[i - 1], mod)


def _alias_module(old: str, new_mod) -> None:
    _ensure_parents(old)
    sys.modules[old] = new_mod
    parent, child = old.rsplit(".", 1)
    setattr(sys.modules[parent], child, new_mod)


def install(alias_top_level: bool = False, quiet: bool = False) -> None:
    roots = [_PKG] + (["physicsnemo"] if alias_top_level else [])
    if alias_top_level and "physicsnemo" not in sys.modules:
        sys.modules["physicsnemo"] = importlib.import_module(_PKG)
    for root in roots:
        for old, new in COMPAT_MAP.items():
            try:
                target = importlib.import_module(f"{_PKG}.{new}")
            except ImportError:
                warnings.warn(f"Failed to import new module '{_PKG}.{new}' for compat alias '{root}.{old}'")
                continue
            _alias_module(f"{root}.{old}", target)
            if not quiet:
                warnings.warn(f"[compat] {root}.{old} is moved; use {_PKG}.{new} instead", DeprecationWarning)
        for old, new in OBJECT_COMPAT_MAP.items():
            new_mod, new_obj = new.rsplit(".", 1)
            old_mod, old_obj = f"{root}.{old}".rsplit(".", 1)
            try:
                obj = getattr(importlib.import_module(f"{_PKG}.{new_mod}"), new_obj)
            except (ImportError, AttributeError):
                continue
            if old_mod not in sys.modules:
                _ensure_parents(old_mod + ".x")
                if old_mod not in sys.modules:
                    sys.modules[old_mod] = types.ModuleType(old_mod)
            setattr(sys.modules[old_mod], old_obj, obj)


__all__ = ["install", "COMPAT_MAP", "OBJECT_COMPAT_MAP"]
