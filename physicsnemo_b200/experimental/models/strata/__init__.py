"""Strata: 3-D transformer regressors for fields on the sphere (backbone ``StrataTransformer3D``, two-stage ``Strata``)."""

from .strata import Strata
from .transformer import StrataTransformer3D

__all__ = ["Strata", "StrataTransformer3D"]
