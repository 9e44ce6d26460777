"""VFGN (Virtual Foundry Graph Net) model."""
from .graph_network_modules import VFGNLearnedSimulator

__all__ = ["VFGNLearnedSimulator"]
