from .legacy_generate import diffusion_step, regression_step

__all__ = ["diffusion_step", "regression_step"]
