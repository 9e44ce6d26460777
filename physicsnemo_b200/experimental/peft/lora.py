"""Low-rank adaptation (LoRA) of trained models: wrap selected Linear-like layers, train only the adapters, save / load
them as a small archive, merge them back into the base weights.

Parity: ``physicsnemo/experimental/peft/`` (``config.py``, ``lora.py``, ``apply.py``, ``merge.py``, ``io.py``, ``utils.py``).
Adapter archives use the reference's layout: a stored zip with ``adapter_model.pt`` (the trainable tensors),
``adapter_config.json`` and ``metadata.json`` (format version, kind, base fingerprint).
"""
from __future__ import annotations

import datetime
import hashlib
import io
import json
import logging
import math
import re
import zipfile
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Literal, Union

import torch
import torch.nn as nn

logger = logging.getLogger("experimental.peft")
LoRAInit = Union[Literal["default"], Callable[[torch.Tensor], None]]


@dataclass
class LoRAConfig:
    """Exactly one selector: ``target_modules`` (names), ``target_pattern`` (regex on names) or ``target_filter``."""

    rank: int = 16
    alpha: float | None = None
    target_modules: list[str] | None = None
    target_pattern: str | None = None
    target_filter: Callable[[str, nn.Module], bool] | None = None
    lora_dropout: float = 0.0
    extras_trainable: list[str] = field(default_factory=list)
    wrap_mlp: bool = False
    init: LoRAInit = "default"

    def __post_init__(self) -> None:
        chosen = [k for k in ("target_modules", "target_pattern", "target_filter") if getattr(self, k) is not None]
        if len(chosen) != 1:
            raise ValueError(f"Exactly one of target_modules, target_pattern, target_filter must be set, got {len(chosen)} ({chosen}).")
        if self.target_modules is not None and len(self.target_modules) == 0:
            raise ValueError("target_modules is an empty list — nothing to select.")
        if self.target_pattern == "":
            raise ValueError("target_pattern is an empty string — nothing to select.")
        if self.rank <= 0:
            raise ValueError(f"rank must be a positive integer, got {self.rank}.")
        if not 0.0 <= self.lora_dropout < 1.0:
            raise ValueError(f"lora_dropout must be in [0.0, 1.0), got {self.lora_dropout}.")
        if not (callable(self.init) or self.init == "default"):
            raise ValueError(f"init={self.init!r} is not supported; use 'default' or a callable that initializes the lora_A tensor in place.")

    @property
    def effective_alpha(self) -> float:
        return float(self.alpha) if self.alpha is not None else float(self.rank)

    @property
    def scaling(self) -> float:
        return self.effective_alpha / self.rank


class LoRALayer:
    """Mixin of every adapter: factors ``lora_A [in, r]``, ``lora_B [r, out]`` (zero), ``delta(x) = drop(x) A B · α/r``."""

    mergeable: bool = False

    def _make_lora_params(self, in_features, out_features, ref_weight, rank, alpha, dropout, init: LoRAInit = "default") -> None:
        self.rank, self.alpha, self.scaling, self.enabled = rank, alpha, alpha / rank, True
        self.lora_A = nn.Parameter(torch.empty(in_features, rank, device=ref_weight.device, dtype=ref_weight.dtype))
        self.lora_B = nn.Parameter(torch.zeros(rank, out_features, device=ref_weight.device, dtype=ref_weight.dtype))
        self.lora_dropout = nn.Dropout(p=dropout) if dropout > 0.0 else nn.Identity()
        if callable(init):
            init(self.lora_A)
        elif init == "default":
            nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        else:
            raise ValueError(f"unknown init strategy {init!r}; use 'default' or a callable.")

    def lora_delta(self, x: torch.Tensor) -> torch.Tensor:
        return self.lora_dropout(x) @ self.lora_A @ self.lora_B * self.scaling

    @classmethod
    def is_compatible(cls, base_layer: nn.Module) -> bool:
        return True


class LoRALinear(nn.Module, LoRALayer):
    """Adapter around an ``nn.Linear``-like layer (``in_features`` / ``out_features`` or a 2-D ``weight``)."""

    mergeable = True

    def __init__(self, base_layer: nn.Module, rank: int, alpha: float, dropout: float = 0.0, init: LoRAInit = "default") -> None:
        nn.Module.__init__(self)
        if not self.is_compatible(base_layer):
            raise TypeError(f"{type(base_layer).__name__} is not Linear-like (no in_features/out_features and no 2-D weight)")
        self.base_layer = base_layer
        for p in base_layer.parameters():
            p.requires_grad = False
        fin, fout = getattr(base_layer, "in_features", None), getattr(base_layer, "out_features", None)
        if fin is None or fout is None:
            fout, fin = base_layer.weight.shape
        self._make_lora_params(int(fin), int(fout), base_layer.weight, rank, alpha, dropout, init)

    @classmethod
    def is_compatible(cls, base_layer: nn.Module) -> bool:
        if getattr(base_layer, "in_features", None) is not None and getattr(base_layer, "out_features", None) is not None:
            return True
        return getattr(getattr(base_layer, "weight", None), "ndim", None) == 2

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = self.base_layer(x)
        return out + self.lora_delta(x) if self.enabled else out

    @torch.no_grad()
    def merge_into_base(self) -> None:
        delta = (self.lora_A.float() @ self.lora_B.float()).t() * self.scaling
        self.base_layer.weight.add_(delta.to(self.base_layer.weight.dtype))


_LORA_WRAPPERS: dict[type, Callable[..., nn.Module]] = {nn.Linear: LoRALinear}


def register_lora_wrapper(layer_type: type, wrapper_factory: Callable[..., nn.Module]) -> None:
    _LORA_WRAPPERS[layer_type] = wrapper_factory


def get_wrapper_for(module: nn.Module):
    for cls in type(module).__mro__:
        if cls in _LORA_WRAPPERS:
            return _LORA_WRAPPERS[cls]
    return None


def wrappable_types() -> tuple[type, ...]:
    return tuple(_LORA_WRAPPERS)


def is_lora_layer(module: nn.Module) -> bool:
    return isinstance(module, LoRALayer)


# ---- apply / merge ---------------------------------------------------------------------------------------------------
@dataclass
class ApplyResult:
    n_wrapped: int
    n_trainable: int
    n_frozen: int
    trainable_names: list[str] = field(default_factory=list)
    base_fingerprint: str = ""


def compute_base_fingerprint(model: nn.Module) -> str:
    """Hash of the module tree (names, types) and the state-dict shapes: identifies the architecture, not the values."""
    h = hashlib.sha256()
    for name, module in model.named_modules():
        h.update(f"{name}:{type(module).__name__}\n".encode())
    for key, tensor in model.state_dict().items():
        h.update(f"{key}:{tuple(tensor.shape)}\n".encode())
    return h.hexdigest()


_MLP_TARGET_PATTERNS = [r"\.ln_mlp1$", r"\.ln_mlp1\.\d+\.layers\.\d+$"]


def resolve_targets(model: nn.Module, config: LoRAConfig) -> list[tuple]:
    """``(name, parent, child_name, module)`` of every layer the config selects and a registered wrapper can adapt."""
    if config.target_modules is not None:
        names = set(config.target_modules)
        matcher = lambda n, m: n in names  # noqa: E731
    elif config.target_pattern is not None:
        pat = re.compile(config.target_pattern)
        matcher = lambda n, m: pat.search(n) is not None  # noqa: E731
    else:
        matcher = config.target_filter
    mlp = [re.compile(p) for p in _MLP_TARGET_PATTERNS] if config.wrap_mlp else []
    modules = dict(model.named_modules())
    targets = []
    for name, module in modules.items():
        if name == "" or is_lora_layer(module):
            continue
        wrapper = get_wrapper_for(module)
        hit = matcher(name, module)
        if wrapper is None:
            if hit:
                logger.warning("LoRA selector matched %s (%s), but no wrapper is registered for that type; skipping it.", name, type(module).__name__)
            continue
        if not (hit or any(p.search(name) for p in mlp)):
            continue
        compatible = getattr(wrapper, "is_compatible", None)
        if compatible is not None and not compatible(module):
            continue
        parent_name, _, child = name.rpartition(".")
        targets.append((name, modules[parent_name] if parent_name else model, child, module))
    return targets


def apply_lora(model: nn.Module, config: LoRAConfig, compute_fingerprint: bool = True) -> ApplyResult:
    if any(is_lora_layer(m) for m in model.modules()):
        raise ValueError("model already contains LoRA layers; apply_lora is not re-entrant. Start from a fresh base model (or call merge_lora first).")
    fingerprint = compute_base_fingerprint(model) if compute_fingerprint else ""
    targets = resolve_targets(model, config)
    if not targets:
        raise ValueError("apply_lora matched 0 wrappable layers. Check target_modules / target_pattern / target_filter.")
    for _name, parent, child, module in targets:
        wrapped = get_wrapper_for(module)(module, rank=config.rank, alpha=config.effective_alpha, dropout=config.lora_dropout, init=config.init)
        if not is_lora_layer(wrapped):
            raise TypeError(f"LoRA wrapper for {type(module).__name__} returned a {type(wrapped).__name__}, which does not subclass LoRALayer.")
        setattr(parent, child, wrapped)
    for p in model.parameters():
        p.requires_grad = False
    base_ids = set()
    for m in model.modules():
        if is_lora_layer(m):
            m.lora_A.requires_grad = m.lora_B.requires_grad = True
            base_ids.update(id(p) for p in m.base_layer.parameters())
    extras = set(config.extras_trainable)
    for name, m in model.named_modules():
        if name in extras:
            for p in m.parameters():
                if id(p) not in base_ids:
                    p.requires_grad = True
    model._lora_base_fingerprint = fingerprint
    model._lora_adapter_config = {"rank": config.rank, "alpha": config.effective_alpha, "lora_dropout": config.lora_dropout,
                                  "extras_trainable": list(config.extras_trainable), "init": config.init if isinstance(config.init, str) else "custom"}
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    return ApplyResult(n_wrapped=len(targets), n_trainable=sum(p.numel() for p in model.parameters() if p.requires_grad),
                       n_frozen=sum(p.numel() for p in model.parameters() if not p.requires_grad), trainable_names=trainable,
                       base_fingerprint=fingerprint)


def merge_lora(model: nn.Module) -> nn.Module:
    """Fold every mergeable adapter into its base layer and put the base layer back in place."""
    for name, module in list(model.named_modules()):
        if not is_lora_layer(module) or not getattr(module, "mergeable", True):
            continue
        module.merge_into_base()
        parent_name, _, child = name.rpartition(".")
        setattr(model.get_submodule(parent_name) if parent_name else model, child, module.base_layer)
    return model


# ---- archive ---------------------------------------------------------------------------------------------------------
_FORMAT_VERSION, _KIND = 1, "lora_adapter"
_FILES = ("adapter_config.json", "adapter_model.pt", "metadata.json")


def save_adapter(model: nn.Module, path: str | Path) -> None:
    meta = getattr(model, "_lora_adapter_config", None)
    if meta is None:
        raise ValueError("model has no stashed LoRA config; call apply_lora(model, config) before save_adapter.")
    wrapped = [n for n, m in model.named_modules() if is_lora_layer(m)]
    if not wrapped:
        raise ValueError("no LoRA layers found in model; cannot save an adapter (after merge_lora save a full checkpoint instead).")
    cfg = {"rank": meta["rank"], "alpha": meta["alpha"], "lora_dropout": meta["lora_dropout"], "target_modules": wrapped,
           "extras_trainable": list(meta["extras_trainable"]), "init": meta["init"]}
    from ... import __version__ as version

    metadata = {"format_version": _FORMAT_VERSION, "kind": _KIND, "physicsnemo_version": version, "torch_version": torch.__version__,
                "base_fingerprint": getattr(model, "_lora_base_fingerprint", ""), "n_wrapped": len(wrapped),
                "created": datetime.datetime.now(datetime.timezone.utc).isoformat()}
    buf = io.BytesIO()
    torch.save({n: p.detach().cpu() for n, p in model.named_parameters() if p.requires_grad}, buf)
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    with zipfile.ZipFile(str(path), "w", zipfile.ZIP_STORED) as z:
        z.writestr("adapter_model.pt", buf.getvalue())
        z.writestr("adapter_config.json", json.dumps(cfg, indent=2))
        z.writestr("metadata.json", json.dumps(metadata, indent=2))


def load_adapter(model: nn.Module, path: str | Path, strict: bool = True) -> None:
    with zipfile.ZipFile(str(path), "r") as z:
        missing = [f for f in _FILES if f not in set(z.namelist())]
        if missing:
            raise IOError(f"{path} is missing adapter files {missing}.")
        metadata, cfg, state_bytes = json.loads(z.read("metadata.json")), json.loads(z.read("adapter_config.json")), z.read("adapter_model.pt")
    if metadata.get("kind") != _KIND:
        raise ValueError(f"{path} is not a LoRA adapter (kind={metadata.get('kind')!r}).")
    saved, current = metadata.get("base_fingerprint", ""), compute_base_fingerprint(model)
    if saved and saved != current:
        msg = f"base fingerprint mismatch: adapter was trained on a different base model (adapter={saved}, this model={current})."
        if strict:
            raise ValueError(msg + " Pass strict=False to load anyway.")
        logger.warning(msg)
    apply_lora(model, LoRAConfig(rank=cfg["rank"], alpha=cfg["alpha"], lora_dropout=cfg.get("lora_dropout", 0.0), target_modules=cfg["target_modules"],
                                 extras_trainable=cfg.get("extras_trainable", [])))
    state = torch.load(io.BytesIO(state_bytes), map_location="cpu", weights_only=True)
    unexpected = list(model.load_state_dict(state, strict=False).unexpected_keys)
    if unexpected:
        raise RuntimeError(f"adapter contains keys not present after re-applying LoRA: {unexpected[:8]}. The adapter and base model are incompatible.")


# ---- utilities -------------------------------------------------------------------------------------------------------
def split_params_for_optimizer(model: nn.Module) -> dict[str, list]:
    lora = [p for m in model.modules() if is_lora_layer(m) for p in (m.lora_A, m.lora_B)]
    ids = {id(p) for p in lora}
    rest = [p for p in model.parameters() if id(p) not in ids]
    return {"lora": lora, "extras": [p for p in rest if p.requires_grad], "frozen": [p for p in rest if not p.requires_grad]}


def print_trainable_parameters(model: nn.Module, use_logger: bool = False) -> str:
    trainable, total = sum(p.numel() for p in model.parameters() if p.requires_grad), sum(p.numel() for p in model.parameters())
    msg = f"trainable params: {trainable:,} ({100.0 * trainable / total if total else 0.0:.2f}% of {total:,} total)"
    (logger.info if use_logger else print)(msg)
    return msg


def set_adapter_enabled(model: nn.Module, enabled: bool) -> None:
    for m in model.modules():
        if is_lora_layer(m):
            m.enabled = enabled
