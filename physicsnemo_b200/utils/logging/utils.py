"""Logging helpers (parity: ``physicsnemo/utils/logging/utils.py:24-61``)."""
from datetime import datetime

import torch

from ...distributed.manager import DistributedManager


def create_ddp_group_tag(group_name: str = None) -> str:
    """A tag shared by all ranks of a job: ``{group_name}_{rank-0 start time}`` (broadcast from rank 0)."""
    dist = DistributedManager()
    if dist.rank == 0:
        tag = (group_name + "_" if group_name else "") + datetime.now().astimezone().strftime("%m%d%y_%H-%M-%S")
        codes = [ord(c) for c in tag]
    else:
        codes = []
    if dist.distributed and torch.distributed.is_initialized() and dist.world_size > 1:
        obj = [codes]
        torch.distributed.broadcast_object_list(obj, src=0)
        codes = obj[0]
    return "".join(chr(c) for c in codes)
