"""``FunctionSpec``: one public functional, one sm_100a kernel, one oracle.

Parity: ``physicsnemo/core/function_spec.py`` — ``register`` decorator
(``:229-297``), ``make_function`` producing the public callable with an
``implementation=`` keyword (``:400-478``), ``dispatch`` (``:480-533``),
benchmark hooks ``make_inputs_forward/backward`` and ``compare_forward/backward``.

Design here: every functional carries at most two implementations — ``"cuda"``
(the hand-written sm_100a kernel, chosen whenever the first tensor argument
lives on a CUDA device and the native extension is loaded) and ``"torch"``
(plain PyTorch; the CPU path and the numerical oracle of the kernel).  There is
no ranking across third-party back ends; ``rank`` is kept for API parity and
only orders implementations that are usable for the given device.
"""
from __future__ import annotations

import importlib.util
import inspect
import warnings
from dataclasses import dataclass
from typing import Callable, Dict, Sequence

import torch


@dataclass
class Implementation:
    name: str
    func: Callable
    required_imports: tuple
    rank: int
    baseline: bool
    available: bool
    device_types: tuple  # device types this implementation can run on; () = any


class FunctionSpec:
    """Base class; subclasses decorate static methods with ``register``."""

    _registry: Dict[str, Dict[str, Implementation]] = {}
    _warned: set = set()

    # ------------------------------------------------------------ registry
    @classmethod
    def _class_key(cls) -> str:
        return f"{cls.__module__}.{cls.__qualname__}"

    @staticmethod
    def _check_imports(imports: Sequence[str]) -> bool:
        for spec in imports:
            name = spec.split(">")[0].split("=")[0].split("<")[0].strip()
            try:
                if importlib.util.find_spec(name) is None:
                    return False
            except (ImportError, ValueError):
                return False
        return True

    @classmethod
    def register(
        cls,
        name: str,
        required_imports: Sequence[str] | None = None,
        rank: int = 0,
        baseline: bool = False,
        device_types: Sequence[str] | None = None,
    ):
        """Decorator used inside a subclass body to add an implementation."""

        def decorator(func):
            target = func.__func__ if isinstance(func, (staticmethod, classmethod)) else func
            qualname = getattr(target, "__qualname__", "")
            if "." not in qualname:
                raise ValueError("FunctionSpec.register must be used inside a class body")
            key = f"{target.__module__}.{qualname.rsplit('.', 1)[0]}"
            imports = tuple(required_imports or ())
            devs = tuple(device_types) if device_types is not None else (("cuda",) if name == "cuda" else ())
            impl = Implementation(name, target, imports, rank, baseline, FunctionSpec._check_imports(imports), devs)
            table = FunctionSpec._registry.setdefault(key, {})
            if name in table:
                raise ValueError(f"Implementation '{name}' already registered for {key}")
            table[name] = impl
            return staticmethod(target)

        return decorator

    @classmethod
    def _get_impls(cls) -> Dict[str, Implementation]:
        return FunctionSpec._registry.get(cls._class_key(), {})

    @classmethod
    def implementations(cls):
        """Names of registered implementations, best first."""
        return tuple(i.name for i in sorted(cls._get_impls().values(), key=lambda i: i.rank))

    @classmethod
    def available_implementations(cls):
        return tuple(i.name for i in sorted(cls._get_impls().values(), key=lambda i: i.rank) if i.available)

    @classmethod
    def baseline_implementation(cls) -> str:
        impls = cls._get_impls()
        for i in impls.values():
            if i.baseline:
                return i.name
        return "torch" if "torch" in impls else sorted(impls.values(), key=lambda i: -i.rank)[0].name

    # ------------------------------------------------------------ dispatch
    @staticmethod
    def _first_device(args, kwargs) -> str:
        for a in list(args) + list(kwargs.values()):
            if isinstance(a, torch.Tensor):
                return a.device.type
            if isinstance(a, (list, tuple)):
                for b in a:
                    if isinstance(b, torch.Tensor):
                        return b.device.type
        return "cpu"

    @classmethod
    def dispatch(cls, *args, **kwargs):
        implementation = kwargs.pop("implementation", None)
        impls = cls._get_impls()
        if not impls:
            raise NotImplementedError(f"{cls.__name__} has no implementations")
        if implementation is not None:
            if implementation not in impls:
                raise ValueError(
                    f"Unknown implementation '{implementation}' for {cls.__name__}; choose from {tuple(impls)}"
                )
            impl = impls[implementation]
            if not impl.available:
                raise ImportError(f"Implementation '{implementation}' is not available for {cls.__name__}")
            return impl.func(*args, **kwargs)
        dev = cls._first_device(args, kwargs)
        usable = [
            i for i in impls.values() if i.available and (not i.device_types or dev in i.device_types)
        ]
        if not usable:
            raise ImportError(f"No implementation of {cls.__name__} can run on device type '{dev}'")
        return sorted(usable, key=lambda i: i.rank)[0].func(*args, **kwargs)

    @classmethod
    def make_function(cls, name: str | None = None):
        """Build the public function (adds a keyword-only ``implementation``)."""

        def _function(*args, **kwargs):
            # sharded inputs: these functions are not torch functions, so ``__torch_function__`` never sees them; the
            # domain-parallel layer registers its rules by name instead (``ShardTensor.register_named_function_handler``)
            sharded = next((a for a in (*args, *kwargs.values()) if type(a).__name__ == "ShardTensor"), None)
            if sharded is not None:
                from ..parallel import patches  # noqa: F401  (registers the rules on first use)

                registry = type(sharded)._named_function_registry
                handler = registry.get(f"{cls.__module__}.{_function.__name__}") or registry.get(_function.__name__)
                if handler is None:
                    from ..parallel.shard_tensor import MissingShardPatch

                    raise MissingShardPatch(f"no ShardTensor rule is registered for '{_function.__name__}'")
                return handler(_function, (type(sharded),), args, kwargs)
            return cls.dispatch(*args, **kwargs)

        impls = cls._get_impls()
        if impls:
            src = impls.get("torch") or sorted(impls.values(), key=lambda i: i.rank)[0]
            try:
                sig = inspect.signature(src.func)
                params = list(sig.parameters.values())
                if "implementation" not in sig.parameters:
                    at = next((i for i, p in enumerate(params) if p.kind is inspect.Parameter.VAR_KEYWORD), len(params))
                    params.insert(at, inspect.Parameter("implementation", inspect.Parameter.KEYWORD_ONLY, default=None))
                    sig = sig.replace(parameters=params)
                _function.__signature__ = sig
            except (TypeError, ValueError):
                pass
        _function.__name__ = name or cls.__name__
        _function.__qualname__ = _function.__name__
        _function.__module__ = cls.__module__
        _function.__doc__ = cls.__doc__
        _function.spec = cls
        return _function

    # ------------------------------------------------ benchmark/test hooks
    @classmethod
    def make_inputs_forward(cls, device="cpu"):
        """Yield ``(label, args, kwargs)`` cases; subclasses override."""
        return iter(())

    @classmethod
    def make_inputs_backward(cls, device="cpu"):
        for label, args, kwargs in cls.make_inputs_forward(device):
            args = tuple(
                a.detach().clone().requires_grad_(True) if isinstance(a, torch.Tensor) and a.is_floating_point() else a
                for a in args
            )
            yield label, args, kwargs

    @classmethod
    def compare_forward(cls, out, ref, rtol=1e-4, atol=1e-5):
        outs = out if isinstance(out, (tuple, list)) else (out,)
        refs = ref if isinstance(ref, (tuple, list)) else (ref,)
        for o, r in zip(outs, refs):
            if isinstance(o, torch.Tensor):
                torch.testing.assert_close(o.float().cpu(), r.float().cpu(), rtol=rtol, atol=atol)

    @classmethod
    def compare_backward(cls, grads, ref_grads, rtol=1e-3, atol=1e-4):
        cls.compare_forward(grads, ref_grads, rtol=rtol, atol=atol)
