from .domain_parallel import DomainParallelNoiseScheduler
from .schedulers import (EDMLogUniformNoiseScheduler, EDMNoiseScheduler, IDDPMNoiseScheduler,
                         LinearGaussianNoiseScheduler, NoiseScheduler, StudentTEDMNoiseScheduler, VENoiseScheduler,
                         VPNoiseScheduler)

__all__ = ["NoiseScheduler", "LinearGaussianNoiseScheduler", "EDMNoiseScheduler", "EDMLogUniformNoiseScheduler",
           "VPNoiseScheduler", "VENoiseScheduler", "IDDPMNoiseScheduler", "StudentTEDMNoiseScheduler",
           "DomainParallelNoiseScheduler"]
