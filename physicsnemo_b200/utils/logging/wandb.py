"""Weights & Biases initialisation helper (parity: ``physicsnemo/utils/logging/wandb.py:42-125``); optional."""
import logging
import os
from datetime import datetime
from pathlib import Path
from typing import Literal, Optional

from ...distributed.manager import DistributedManager
from .utils import create_ddp_group_tag

DEFAULT_WANDB_CONFIG = "~/.netrc"
logger = logging.getLogger(__name__)
_WANDB_START_TIME = datetime.now().astimezone()


def initialize_wandb(project: str, entity: str, name: str = "train", group: Optional[str] = None,
                     sync_tensorboard: bool = False, save_code: bool = False, resume: Optional[str] = None,
                     wandb_id: Optional[str] = None, config=None, mode: Literal["offline", "online", "disabled"] = "offline",
                     results_dir: Optional[str] = None, init_timeout: int = 90):
    """Start a W&B run named per rank (``{name}_Process_{rank}_{time}``) and enable the LaunchLogger back end."""
    import wandb

    from .launch import LaunchLogger

    if results_dir is None:
        results_dir = str(Path("./wandb").absolute())
    wandb_dir = results_dir
    if DistributedManager.is_initialized() and DistributedManager().distributed:
        if group is None:
            group = create_ddp_group_tag()
        start_time = datetime.now().astimezone()
        wandb_name = f"{name}_Process_{DistributedManager().rank}_{start_time.strftime('%m/%d/%y_%H:%M:%S')}"
    else:
        start_time = datetime.now().astimezone()
        wandb_name = f"{name}_{start_time.strftime('%m/%d/%y_%H:%M:%S')}"
    os.makedirs(wandb_dir, exist_ok=True)
    wandb.init(project=project, entity=entity, sync_tensorboard=sync_tensorboard, name=wandb_name, resume=resume,
               config=config, mode=mode, dir=wandb_dir, group=group, save_code=save_code, id=wandb_id,
               settings=wandb.Settings(init_timeout=init_timeout))
    LaunchLogger.toggle_wandb(True)


def alert(title, text, duration=300, level=0, is_master=True):
    import wandb

    levels = {0: wandb.AlertLevel.INFO, 1: wandb.AlertLevel.WARN, 2: wandb.AlertLevel.ERROR}
    if is_master and wandb.run is not None:
        wandb.alert(title=title, text=text, level=levels[level], wait_duration=duration)
