"""MLflow initialisation helper (parity: ``physicsnemo/utils/logging/mlflow.py:42-170``); optional."""
import os
from datetime import datetime
from pathlib import Path
from typing import Literal, Optional, Tuple

from ...distributed.manager import DistributedManager
from .utils import create_ddp_group_tag


def initialize_mlflow(experiment_name: str, experiment_desc: Optional[str] = None, run_name: Optional[str] = None,
                      run_desc: Optional[str] = None, user_name: Optional[str] = None,
                      mode: Literal["offline", "online", "ngc"] = "offline", tracking_location: Optional[str] = None,
                      artifact_location: Optional[str] = None) -> Tuple:
    """Create / reuse an MLflow experiment and start a per-rank run; returns ``(client, run)``."""
    import mlflow
    from mlflow.tracking import MlflowClient

    from .launch import LaunchLogger

    dist = DistributedManager() if DistributedManager.is_initialized() else None
    if dist is not None and dist.rank != 0:
        return None, None
    start_time = datetime.now().astimezone().strftime("%m/%d/%y %H:%M:%S")
    group_name = create_ddp_group_tag(run_name) if (dist and dist.distributed) else start_time
    run_name = f"{run_name} {group_name}" if run_name else group_name
    if mode == "online":
        tracking_uri = tracking_location or "http://localhost:5000"
    else:
        tracking_uri = tracking_location or f"file://{Path('./mlflow_output').resolve()}"
    mlflow.set_tracking_uri(tracking_uri)
    client = MlflowClient()
    exp = client.get_experiment_by_name(experiment_name)
    exp_id = exp.experiment_id if exp is not None else client.create_experiment(experiment_name, artifact_location=artifact_location)
    if experiment_desc:
        client.set_experiment_tag(exp_id, "mlflow.note.content", experiment_desc)
    run = client.create_run(exp_id, tags={"mlflow.user": user_name}, run_name=run_name)
    if run_desc:
        client.set_tag(run.info.run_id, "mlflow.note.content", run_desc)
    LaunchLogger.mlflow_run, LaunchLogger.mlflow_client = run, client
    LaunchLogger.toggle_mlflow(True)
    return client, run
