"""ONNX export and ONNX-Runtime inference helpers (parity: ``physicsnemo/deploy/onnx/utils.py``).

Export traces the model on CPU in plain PyTorch ops (the fused sm_100a kernels are bypassed there, the
PyTorch formulation being numerically equivalent), opset 15, and restores the model's device afterwards.
"""
import io
import logging
from typing import Tuple, Union

import torch
import torch.nn as nn

from ...core.version_check import OptionalImport

ort = OptionalImport("onnxruntime")
Tensor = torch.Tensor
logger = logging.getLogger(__name__)


def check_ort_install(func):
    def wrapper(*args, **kwargs):
        if not ort.available:
            raise ModuleNotFoundError("ONNXRuntime is not installed. 'pip install onnxruntime onnxruntime_gpu'")
        return func(*args, **kwargs)

    wrapper.__name__, wrapper.__doc__ = func.__name__, func.__doc__
    return wrapper


def export_to_onnx_stream(model: nn.Module, invars: Union[Tensor, Tuple[Tensor, ...]], verbose: bool = False) -> bytes:
    """Serialised ONNX graph of ``model`` traced on ``invars``."""
    args = (invars,) if isinstance(invars, Tensor) else tuple(invars)
    args = tuple(a.detach().cpu() for a in args)
    if hasattr(model, "device"):
        home = model.device
    else:
        first = next(model.parameters(), None)
        home = first.device if first is not None else "cpu"
    buf = io.BytesIO()
    try:
        try:
            torch.onnx.export(model.cpu(), args, buf, opset_version=15, verbose=verbose, dynamo=False)
        except TypeError:  # older exporters do not know the ``dynamo`` switch
            torch.onnx.export(model.cpu(), args, buf, opset_version=15, verbose=verbose)
    finally:
        model.to(home)
    return buf.getvalue()


@check_ort_install
def get_ort_session(model: Union[bytes, str], device: torch.device = "cuda"):
    """``onnxruntime.InferenceSession`` with the CUDA provider first when ``device`` is a CUDA device."""
    providers = ["CPUExecutionProvider"]
    if "cuda" in str(device):
        providers.insert(0, "CUDAExecutionProvider")
    return ort.InferenceSession(model, providers=providers)


@check_ort_install
def run_onnx_inference(model: Union[bytes, str], invars: Union[Tensor, Tuple[Tensor, ...]],
                       device: torch.device = "cuda") -> Tuple[Tensor]:
    sess = get_ort_session(model, device)
    args = (invars,) if isinstance(invars, Tensor) else tuple(invars)
    feed = {spec.name: a.detach().cpu().numpy() for spec, a in zip(sess.get_inputs(), args)}
    return tuple(torch.Tensor(o) for o in sess.run(None, feed))
