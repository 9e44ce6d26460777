from .super_res_net import SRResNet
