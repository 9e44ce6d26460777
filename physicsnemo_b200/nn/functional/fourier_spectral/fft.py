"""Real FFTs that also export to ONNX.

Parity: ``physicsnemo/nn/functional/fourier_spectral/fft.py`` — outside an ONNX export the functions
are ``torch.fft``; during export complex tensors are carried as a trailing real dimension of
size 2 and the transforms become the ``com.microsoft::Rfft`` / ``Irfft`` contrib operators
(un-normalised, one-sided, last 1 or 2 axes), with axis permutation and ``norm`` scaling applied
around them.  Padding / trimming (``n`` / ``s`` different from the input size) is not exportable.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
from torch import Tensor
from torch.autograd import Function

from ....core.function_spec import FunctionSpec


def _exporting() -> bool:
    return torch.onnx.is_in_onnx_export()


def _is_last_dims(dim: Tuple[int, ...], inp_ndim: int) -> bool:
    return all(d % inp_ndim == inp_ndim - len(dim) + i for i, d in enumerate(dim))


def _no_resize(what: str, sizes, dim, inp_sizes) -> RuntimeError:
    return RuntimeError(f"Padding/trimming is not yet supported, got sizes {sizes}, DFT dims {dim}, input dims {inp_sizes}{what}.")


def _check_padding_rfft(sizes, dim, inp_sizes) -> None:
    if len(sizes) != len(dim):
        raise ValueError(f"{sizes}, {dim}")
    for s, d in zip(sizes, dim):
        if s is not None and s >= 0 and s != inp_sizes[d]:
            raise _no_resize("", sizes, dim, inp_sizes)


def _check_padding_irfft(sizes, dim, inp_sizes) -> None:
    if len(sizes) != len(dim):
        raise ValueError(f"{sizes}, {dim}")
    for s, d in zip(sizes[:-1], dim[:-1]):
        if s is not None and s >= 0 and s != inp_sizes[d]:
            raise _no_resize("", sizes, dim, inp_sizes)
    last = sizes[-1]
    if last is not None and last > 0 and last != 2 * (inp_sizes[dim[-1]] - 1):
        raise _no_resize(f", expected last size {2 * (inp_sizes[dim[-1]] - 1)}", sizes, dim, inp_sizes)


def _create_axes_perm(ndim: int, dims: Tuple[int, ...]) -> Tuple[List[int], List[int]]:
    """Permutations moving ``dims`` to the trailing axes and back."""
    perm_in = list(range(ndim))
    perm_out = list(perm_in)
    for i in range(-1, -(len(dims) + 1), -1):
        perm_in[dims[i]], perm_in[i] = perm_in[i], perm_in[dims[i]]
    for i in range(-len(dims), 0):
        perm_out[dims[i]], perm_out[i] = perm_out[i], perm_out[dims[i]]
    return perm_in, perm_out


def _norm_name(norm: Optional[str]) -> str:
    norm = "backward" if norm is None else norm
    if norm not in ("forward", "backward", "ortho"):
        raise ValueError(norm)
    return norm


def _scale_output_forward(output: Tensor, norm, sizes, ndim: int) -> Tensor:
    norm = _norm_name(norm)
    if norm == "backward":
        return output
    n = float(math.prod(int(s) for s in sizes[-ndim:]))
    return output / (math.sqrt(n) if norm == "ortho" else n)


def _scale_output_backward(output: Tensor, norm, sizes, ndim: int) -> Tensor:
    norm = _norm_name(norm)
    if norm == "backward":
        return output
    if len(sizes) < ndim + 1:
        raise ValueError
    n = float(math.prod(int(s) for s in sizes[-(ndim + 1):-2]) * 2 * (int(sizes[-2]) - 1))
    return output * (n if norm == "forward" else math.sqrt(n))


def _contrib(g, name: str, inp, ndim: int):
    if ndim not in (1, 2):
        raise ValueError(ndim)
    return g.op(f"com.microsoft::{name}", inp, normalized_i=0, onesided_i=1, signal_ndim_i=ndim)


def _export_only() -> None:
    if not _exporting():
        raise ValueError("Must be called only during ONNX export.")


class OnnxRfft(Function):
    @staticmethod
    def forward(ctx, input: Tensor) -> Tensor:
        _export_only()
        return torch.view_as_real(torch.fft.rfft(input, dim=-1, norm="backward"))

    @staticmethod
    def symbolic(g, input):
        return _contrib(g, "Rfft", input, 1)


class OnnxRfft2(Function):
    @staticmethod
    def forward(ctx, input: Tensor) -> Tensor:
        _export_only()
        return torch.view_as_real(torch.fft.rfft2(input, dim=(-2, -1), norm="backward"))

    @staticmethod
    def symbolic(g, input):
        return _contrib(g, "Rfft", input, 2)


class OnnxIrfft(Function):
    @staticmethod
    def forward(ctx, input: Tensor) -> Tensor:
        _export_only()
        return torch.fft.irfft(torch.view_as_complex(input), dim=-1, norm="backward")

    @staticmethod
    def symbolic(g, input):
        return _contrib(g, "Irfft", input, 1)


class OnnxIrfft2(Function):
    @staticmethod
    def forward(ctx, input: Tensor) -> Tensor:
        _export_only()
        return torch.fft.irfft2(torch.view_as_complex(input), dim=(-2, -1), norm="backward")

    @staticmethod
    def symbolic(g, input):
        return _contrib(g, "Irfft", input, 2)


def _rfft_onnx(input: Tensor, s, dim: Tuple[int, ...], norm) -> Tensor:
    if s is not None:
        _check_padding_rfft(s, dim, input.size())
    ndim = len(dim)
    if ndim not in (1, 2):
        raise ValueError(ndim)
    perm = not _is_last_dims(dim, input.ndim)
    if perm:
        perm_in, perm_out = _create_axes_perm(input.ndim, dim)
        perm_out.append(len(perm_out))
        input = input.permute(perm_in)
    out = (OnnxRfft if ndim == 1 else OnnxRfft2).apply(input)
    out = _scale_output_forward(out, norm, input.size(), ndim)
    return out.permute(perm_out) if perm else out


def _irfft_onnx(input: Tensor, s, dim: Tuple[int, ...], norm) -> Tensor:
    if s is not None:
        _check_padding_irfft(s, dim, input.size())
    ndim = len(dim)
    if ndim not in (1, 2):
        raise ValueError(ndim)
    perm = not _is_last_dims(dim, input.ndim - 1)
    if perm:
        perm_in, perm_out = _create_axes_perm(input.ndim - 1, dim)
        perm_in.append(len(perm_in))
        input = input.permute(perm_in)
    out = (OnnxIrfft if ndim == 1 else OnnxIrfft2).apply(input)
    out = _scale_output_backward(out, norm, input.size(), ndim)
    return out.permute(perm_out) if perm else out


def _pair(value, name: str):
    if value is None:
        return None
    if not (isinstance(value, (tuple, list)) and len(value) == 2):
        raise ValueError(f"{name} must have two entries, got {value}")
    return tuple(value)


class RFFT(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(input, n=None, dim: int = -1, norm=None):
        if not _exporting():
            return torch.fft.rfft(input, n=n, dim=dim, norm=norm)
        if not isinstance(dim, int):
            raise TypeError()
        return _rfft_onnx(input, (n,), (dim,), norm)


class RFFT2(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(input, s=None, dim=(-2, -1), norm=None):
        if not _exporting():
            return torch.fft.rfft2(input, s=s, dim=dim, norm=norm)
        return _rfft_onnx(input, _pair(s, "s"), _pair(dim, "dim"), norm)


class IRFFT(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(input, n=None, dim: int = -1, norm=None):
        if not _exporting():
            return torch.fft.irfft(input, n=n, dim=dim, norm=norm)
        if not isinstance(dim, int):
            raise TypeError()
        return _irfft_onnx(input, (n,), (dim,), norm)


class IRFFT2(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(input, s=None, dim=(-2, -1), norm=None):
        if not _exporting():
            return torch.fft.irfft2(input, s=s, dim=dim, norm=norm)
        return _irfft_onnx(input, _pair(s, "s"), _pair(dim, "dim"), norm)


def _need_pair_axis(t: Tensor) -> None:
    if t.size(-1) != 2:
        raise ValueError("during ONNX export complex tensors are carried as a trailing dimension of size 2")


class ViewAsComplex(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(input):
        if not _exporting():
            return torch.view_as_complex(input)
        _need_pair_axis(input)
        return input


class Real(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(input):
        if not _exporting():
            return input.real
        _need_pair_axis(input)
        return input[..., 0]


class Imag(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(input):
        if not _exporting():
            return input.imag
        _need_pair_axis(input)
        return input[..., 1]


rfft = RFFT.make_function("rfft")
rfft2 = RFFT2.make_function("rfft2")
irfft = IRFFT.make_function("irfft")
irfft2 = IRFFT2.make_function("irfft2")
view_as_complex = ViewAsComplex.make_function("view_as_complex")
real = Real.make_function("real")
imag = Imag.make_function("imag")
