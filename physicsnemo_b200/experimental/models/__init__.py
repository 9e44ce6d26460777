from .tedm import tEDMPrecondSuperRes, tEDMResidualLoss

__all__ = ["tEDMPrecondSuperRes", "tEDMResidualLoss"]
