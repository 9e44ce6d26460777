"""Experimental data pipelines."""
