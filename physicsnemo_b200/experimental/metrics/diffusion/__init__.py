"""Losses of the heavy-tailed (Student-t) EDM variant, under the reference's package path
(``physicsnemo/experimental/metrics/diffusion/loss.py:27``); the class lives beside its preconditioner."""

from ...models.tedm import tEDMResidualLoss

__all__ = ["tEDMResidualLoss"]
