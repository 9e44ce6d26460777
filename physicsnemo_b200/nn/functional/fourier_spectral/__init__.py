from .fft import (IRFFT, IRFFT2, RFFT, RFFT2, Imag, Real, ViewAsComplex, imag, irfft, irfft2, real, rfft, rfft2,
                  view_as_complex)

__all__ = ["IRFFT", "IRFFT2", "RFFT", "RFFT2", "Imag", "Real", "ViewAsComplex", "imag", "irfft", "irfft2", "real", "rfft",
           "rfft2", "view_as_complex"]
