"""The generic rule for operations that act independently of the sharded dimensions.

An operation qualifies when it is point-wise, or when everything it mixes lives in
dimensions that are not sharded (``linear`` / ``layer_norm`` / ``softmax(dim=-1)`` on a tensor
sharded along its token dimension, ...).  Such an operation is applied to the local shards
and the result inherits the placements.  Partial inputs are resolved (all-reduced) first
unless the operation is linear in them.  The reference gets this behaviour from DTensor's
sharding propagation (``physicsnemo/domain_parallel/shard_tensor.py:339-391``).
"""
from __future__ import annotations

import operator
import warnings
from typing import Any, Tuple

import torch
import torch.nn.functional as F
from torch.distributed.tensor import Partial, Replicate, Shard

_NO_TF = torch._C.DisableTorchFunctionSubclass

_META_PROPS = {"shape", "dtype", "device", "ndim", "is_cuda", "layout", "names", "is_sparse", "is_quantized",
               "is_meta", "is_cpu", "itemsize", "nbytes"}
_META_FUNCS = {"size", "dim", "numel", "nelement", "element_size", "is_floating_point", "is_complex", "is_signed",
               "ndimension", "get_device", "is_contiguous", "is_inference", "_is_view", "data_ptr", "__len__",
               "is_shared", "is_pinned", "__hash__", "__format__", "storage_offset"}

_POINTWISE = {
    "add", "sub", "rsub", "mul", "div", "true_divide", "floor_divide", "pow", "neg", "abs", "exp", "exp2", "expm1",
    "log", "log2", "log10", "log1p", "sqrt", "rsqrt", "sin", "cos", "tan", "tanh", "sinh", "cosh", "asin", "acos",
    "atan", "atan2", "sigmoid", "relu", "relu6", "gelu", "silu", "elu", "selu", "celu", "leaky_relu", "softplus",
    "softsign", "hardtanh", "hardswish", "hardsigmoid", "mish", "logsigmoid", "tanhshrink", "softshrink",
    "hardshrink", "threshold", "clamp", "clamp_min", "clamp_max", "clip", "where", "maximum", "minimum", "fmax",
    "fmin", "sign", "square", "reciprocal", "erf", "erfc", "erfinv", "floor", "ceil", "round", "trunc", "frac",
    "lerp", "addcmul", "addcdiv", "nan_to_num", "isnan", "isinf", "isfinite", "eq", "ne", "lt", "le", "gt", "ge",
    "logical_and", "logical_or", "logical_not", "logical_xor", "bitwise_and", "bitwise_or", "bitwise_not",
    "dropout", "alpha_dropout", "feature_alpha_dropout", "to", "type", "float", "half", "bfloat16", "double", "int",
    "long", "bool", "clone", "contiguous", "detach", "zeros_like", "ones_like", "empty_like", "full_like",
    "rand_like", "randn_like", "real", "imag", "conj", "angle", "view_as_real", "view_as_complex", "masked_fill",
    "type_as", "cpu", "cuda", "requires_grad_", "expm1", "sinc", "fmod", "remainder", "copysign", "heaviside",
    "__add__", "__radd__", "__sub__", "__rsub__", "__mul__", "__rmul__", "__truediv__", "__rtruediv__", "__pow__",
    "__rpow__", "__neg__", "__abs__", "__eq__", "__ne__", "__lt__", "__le__", "__gt__", "__ge__", "__and__",
    "__or__", "__invert__", "__floordiv__", "__mod__", "__matmul_scalar__", "polar", "complex", "rrelu", "glu_none",
    "positive", "deg2rad", "rad2deg", "sgn", "logit", "xlogy", "hypot", "logaddexp", "special_expit", "expit",
    "mse_loss_none", "binary_cross_entropy_with_logits_none", "prelu", "softmin_none", "identity",
}
_INPLACE_OK = {n + "_" for n in ("add", "sub", "mul", "div", "clamp", "clamp_min", "clamp_max", "neg", "exp", "sqrt",
                                 "relu", "sigmoid", "tanh", "zero", "fill", "copy", "masked_fill", "pow", "addcmul",
                                 "addcdiv", "lerp", "normal", "uniform", "silu")} | {"__iadd__", "__isub__",
                                                                                    "__imul__", "__itruediv__"}
# functions with a `dim` argument that must not be a sharded dimension
_DIM_FUNCS = {"softmax", "log_softmax", "softmin", "cumsum", "cumprod", "logsumexp", "norm", "normalize", "glu",
              "argmax", "argmin", "max", "min", "amax", "amin", "std", "var", "prod", "sort", "topk", "flip", "roll",
              "cummax", "cummin", "logcumsumexp", "any", "all", "gumbel_softmax", "median", "nanmean", "nansum",
              "fft", "ifft", "rfft", "irfft", "diff", "gather", "index_select", "take_along_dim"}
# functions that mix only trailing feature dimensions
_FEATURE_FUNCS = {"linear": 1, "layer_norm": None, "rms_norm": None, "embedding": 0, "bilinear": 1, "matmul": 1,
                  "mm": 1, "bmm": 1, "einsum": None, "baddbmm": 1, "addmm": 1, "__matmul__": 1, "__rmatmul__": 1,
                  "tensordot": None, "scaled_dot_product_attention": 2}
_LINEAR_IN_PARTIAL = {"mul", "div", "__mul__", "__rmul__", "__truediv__", "neg", "__neg__", "to", "float", "clone",
                      "contiguous", "linear_nobias", "reshape", "view", "permute", "transpose"}


def passthrough(func, args, kwargs) -> Tuple[bool, Any]:
    """Metadata queries are answered by the wrapper itself (global shape / dtype / device)."""
    name = getattr(func, "__name__", "")
    if name == "__get__":
        prop = getattr(getattr(func, "__self__", None), "__name__", None)
        if prop in _META_PROPS:
            with _NO_TF():
                return True, func(*args, **kwargs)
        if prop in ("T", "mT", "H", "mH"):
            t = args[0]
            return True, (t.transpose(-2, -1) if prop in ("mT", "mH") or t.dim() == 2 else t.permute(*reversed(range(t.dim()))))
        if prop == "data":
            return True, args[0].detach()
        if prop == "is_leaf":
            return True, args[0]._local_tensor.is_leaf
    if name in _META_FUNCS:
        with _NO_TF():
            return True, func(*args, **kwargs)
    return False, None


def _shard_args(args, kwargs):
    from .shard_tensor import ShardTensor

    found = []

    def visit(a):
        if isinstance(a, ShardTensor):
            found.append(a)
        elif isinstance(a, (list, tuple)):
            for b in a:
                visit(b)

    for a in args:
        visit(a)
    for a in kwargs.values():
        visit(a)
    return found


def _unwrap(a, resolve_partial: bool, mesh=None):
    from .shard_tensor import ShardTensor
    from .grad_ops import reduce_grad_over_mesh

    if mesh is not None and isinstance(a, torch.Tensor) and not isinstance(a, ShardTensor):
        return reduce_grad_over_mesh(a, mesh)
    if isinstance(a, ShardTensor):
        if resolve_partial and a._spec.is_partial():
            a = a.redistribute(placements=[Replicate() if isinstance(p, Partial) else p for p in a._spec.placements])
        return a._local_tensor
    if isinstance(a, (list, tuple)):
        return type(a)(_unwrap(b, resolve_partial, mesh) for b in a)
    return a


def _norm_dim(d, ndim):
    return d + ndim if d < 0 else d


def apply_local_rule(func, args, kwargs):
    from .shard_tensor import MissingShardPatch, ShardTensor, TensorPromotionMode

    name = getattr(func, "__name__", str(func))
    sts = _shard_args(args, kwargs)
    if not sts:
        with _NO_TF():
            return func(*args, **kwargs)
    ref = max(sts, key=lambda t: (len(t._spec.sharded_tensor_dims()), t.dim()))
    spec = ref._spec
    sharded = spec.sharded_tensor_dims()
    mode = ShardTensor._promotion_mode
    if mode is not TensorPromotionMode.SILENT:
        plain = [a for a in args if isinstance(a, torch.Tensor) and not isinstance(a, ShardTensor)
                 and not isinstance(a, torch.nn.Parameter) and a.dim() > 0]
        if plain:
            if mode is TensorPromotionMode.DISABLED:
                raise RuntimeError(f"{name}: plain tensors cannot be mixed with ShardTensors (promotion disabled)")
            if name not in ShardTensor._warned:
                ShardTensor._warned.add(name)
                warnings.warn(f"{name}: treating a plain tensor as replicated next to a ShardTensor")
    # ---- is the operation safe on local shards?
    ok = name in _POINTWISE or name in _INPLACE_OK
    if not ok and name in _DIM_FUNCS:
        d = kwargs.get("dim", None)
        if d is None:
            pos = [a for a in args[1:] if isinstance(a, int) and not isinstance(a, bool)]
            d = pos[0] if pos else None
        if d is None:
            ok = not sharded  # full reduction over everything needs its own handler
        else:
            dims = d if isinstance(d, (list, tuple)) else [d]
            ok = all(_norm_dim(x, ref.dim()) not in sharded for x in dims)
        if not ok:
            raise MissingShardPatch(f"{name} along a sharded dimension needs a ShardTensor handler")
    if not ok and name in _FEATURE_FUNCS:
        ok = _feature_op_ok(name, ref, sharded, args, kwargs)
    if not ok:
        raise MissingShardPatch(
            f"no ShardTensor rule for '{name}' with placements {spec.placements}; register a handler with "
            "ShardTensor.register_function_handler"
        )
    resolve = name not in _LINEAR_IN_PARTIAL
    largs = tuple(_unwrap(a, resolve, spec.mesh) for a in args)
    lkwargs = {k: _unwrap(v, resolve, spec.mesh) for k, v in kwargs.items()}
    ref_local = ref._local_tensor
    with _NO_TF():
        out = func(*largs, **lkwargs)
    if name in _INPLACE_OK and isinstance(args[0], ShardTensor):
        return args[0]
    return _wrap_like(out, ref, ref_local, name)


def _feature_op_ok(name, ref, sharded, args, kwargs) -> bool:
    nd = ref.dim()
    if name == "layer_norm" or name == "rms_norm":
        ns = args[1] if len(args) > 1 else kwargs.get("normalized_shape")
        k = len(ns) if isinstance(ns, (list, tuple, torch.Size)) else 1
        return all(d < nd - k for d in sharded)
    if name == "einsum":
        return False  # handled by its own patch
    if name == "scaled_dot_product_attention":
        return all(d < nd - 2 for d in sharded)
    if name in ("matmul", "__matmul__", "bmm", "mm", "baddbmm", "addmm", "__rmatmul__"):
        from .shard_tensor import ShardTensor

        ts = [a for a in args if isinstance(a, torch.Tensor)]
        sh = [t for t in ts if isinstance(t, ShardTensor)]
        # every sharded operand must be sharded on batch dims only (not its last two dims)
        return all(all(d < t.dim() - 2 for d in t._spec.sharded_tensor_dims()) or
                   (t is ts[0] and all(d < t.dim() - 1 for d in t._spec.sharded_tensor_dims()) and len(sh) == 1)
                   for t in sh)
    trailing = _FEATURE_FUNCS[name] or 1
    return all(d < nd - trailing for d in sharded)


def _wrap_like(out, ref, ref_local, name):
    from .shard_tensor import MissingShardPatch, ShardTensor
    from .spec import ShardTensorSpec

    if isinstance(out, (tuple, list)):
        return type(out)(_wrap_like(o, ref, ref_local, name) for o in out)
    if not isinstance(out, torch.Tensor):
        return out
    spec = ref._spec
    placements = tuple(Replicate() if isinstance(p, Partial) and name not in _LINEAR_IN_PARTIAL else p
                       for p in spec.placements)
    sharded = [p.dim for p in placements if isinstance(p, Shard)]
    if not sharded:
        return ShardTensor(out, ShardTensorSpec(spec.mesh, placements, out.shape, out.dtype, {}))
    if out.dim() != ref_local.dim() or any(out.shape[d] != ref_local.shape[d] for d in sharded):
        if out.dim() == 0:
            raise MissingShardPatch(f"{name} reduced a sharded tensor to a scalar; use the sharded reductions")
        raise MissingShardPatch(f"{name}: cannot carry the sharding of {spec.placements} to an output of shape "
                                f"{tuple(out.shape)} (input shard {tuple(ref_local.shape)})")
    gshape = list(out.shape)
    for md, p in enumerate(placements):
        if isinstance(p, Shard):
            gshape[p.dim] = spec.global_shape[p.dim]
    return ShardTensor(out, ShardTensorSpec(spec.mesh, placements, torch.Size(gshape), out.dtype,
                                            dict(spec.sharding_sizes)))
