"""Diffusion tool-kit: noise schedulers, preconditioners, losses, samplers, patching."""
from .base import Denoiser, DiffusionModel, Predictor

__all__ = ["Denoiser", "DiffusionModel", "Predictor"]
