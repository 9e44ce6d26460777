"""ONNX-exportable real FFTs (module-level alias of ``nn.functional.fourier_spectral``).

Parity: ``physicsnemo/nn/module/fft.py``.
"""
from ..functional.fourier_spectral.fft import (OnnxIrfft, OnnxIrfft2, OnnxRfft, OnnxRfft2, imag, irfft, irfft2, real, rfft,
                                               rfft2, view_as_complex)

__all__ = ["rfft", "rfft2", "irfft", "irfft2", "real", "imag", "view_as_complex", "OnnxRfft", "OnnxRfft2", "OnnxIrfft",
           "OnnxIrfft2"]
