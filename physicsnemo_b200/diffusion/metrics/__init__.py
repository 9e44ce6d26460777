from .legacy_losses import (EDMLoss, EDMLossLogUniform, EDMLossSR, RegressionLoss, RegressionLossCE, ResidualLoss,
                            VELoss, VPLoss)
from .losses import MSEDSMLoss, WeightedMSEDSMLoss

__all__ = ["MSEDSMLoss", "WeightedMSEDSMLoss", "EDMLoss", "EDMLossLogUniform", "EDMLossSR", "RegressionLoss",
           "RegressionLossCE", "ResidualLoss", "VELoss", "VPLoss"]
