"""Experimental metrics (``metrics.diffusion``: Student-t residual loss)."""
