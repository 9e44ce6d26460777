"""Naming conventions of the symbolic layer.

Parity: ``physicsnemo/sym/constants.py`` — a derivative of ``u`` along ``x`` is the dictionary key
``u__x``; second derivatives repeat the separator (``u__x__y``).
"""
import numpy as np
import torch

diff_str: str = "__"


def diff(y: str, x: str, degree: int = 1) -> str:
    """``diff('u', 'x', 2)`` → ``'u__x__x'``."""
    return diff_str.join([y] + degree * [x])


def split_derivative(name: str):
    """``'u__x__y'`` → ``('u', ['x', 'y'])``; a plain name gives an empty list."""
    head, *wrt = name.split(diff_str)
    return head, wrt


tf_dt = torch.float32
np_dt = np.float32
