"""Capability flags attached to every model.

Parity: ``physicsnemo/core/meta.py:23-66`` (dataclass of optimisation / export
capability flags consulted by the static-capture utilities and the tests).
"""
from __future__ import annotations

from dataclasses import dataclass
import warnings


@dataclass
class ModelMetaData:
    """Describes what a model supports (CUDA graphs, AMP, export paths ...)."""

    # optimisation
    jit: bool = False
    cuda_graphs: bool = False
    amp: bool = False
    amp_cpu: bool | None = None
    amp_gpu: bool | None = None
    torch_fx: bool = False
    # data type
    bf16: bool = False
    # inference
    onnx: bool = False
    onnx_gpu: bool | None = None
    onnx_cpu: bool | None = None
    onnx_runtime: bool = False
    trt: bool = False
    # physics informed
    var_dim: int = -1
    func_torch: bool = False
    auto_grad: bool = False
    # deprecated: the class name is used instead
    name: str | None = None

    def __post_init__(self):
        if self.name is not None:
            warnings.warn(
                "ModelMetaData.name is deprecated; the model class name is used.",
                DeprecationWarning,
                stacklevel=2,
            )
        # the coarse flag fans out to the per-device flags when they are unset
        if self.amp_cpu is None:
            self.amp_cpu = self.amp
        if self.amp_gpu is None:
            self.amp_gpu = self.amp
        if self.onnx_cpu is None:
            self.onnx_cpu = self.onnx
        if self.onnx_gpu is None:
            self.onnx_gpu = self.onnx
