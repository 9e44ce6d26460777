from .preconditioners import (BaseAffinePreconditioner, EDMPreconditioner, IDDPMPreconditioner, VEPreconditioner,
                              VPPreconditioner)
from .legacy import EDMPrecond, EDMPrecondSuperResolution, VEPrecond, VPPrecond, iDDPMPrecond

__all__ = ["BaseAffinePreconditioner", "EDMPreconditioner", "VPPreconditioner", "VEPreconditioner",
           "IDDPMPreconditioner", "EDMPrecond", "EDMPrecondSuperResolution", "VPPrecond", "VEPrecond",
           "iDDPMPrecond"]
