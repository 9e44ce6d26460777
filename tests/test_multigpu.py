"""Multi-GPU checks (2+ B200 in one box): launches ``tests/multigpu_worker.py`` under torchrun.

NVLS is switched off in NCCL for these runs and the package's own kernels use plain peer loads (never ``multimem``),
because one of the checks lets a rank arrive late on purpose.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_multigpu_worker():
    n = min(torch.cuda.device_count(), 4)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29731", os.path.join(root, "tests", "multigpu_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    tail = (proc.stdout + proc.stderr)[-4000:]
    assert proc.returncode == 0 and "MULTIGPU_OK" in proc.stdout, tail
