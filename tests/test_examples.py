"""Every recipe under ``examples/`` runs a few CPU steps with ``--smoke`` (public API end to end)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
RECIPES = ["cfd/darcy_fno/train.py", "cfd/transolver_point_cloud/train.py", "generative/edm_songunet/train.py",
           "cfd/globe_potential_flow/train.py", "cfd/stokes_mgn/train.py", "weather/afno_era5/train.py"]


@pytest.mark.parametrize("recipe", RECIPES)
def test_recipe_smoke(recipe, tmp_path):
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    proc = subprocess.run([sys.executable, str(ROOT / "examples" / recipe), "--smoke", "--out", str(tmp_path / "out")],
                          env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert any((tmp_path / "out").rglob("*.pt")) or any((tmp_path / "out").rglob("*.mdlus")), "the recipe wrote no checkpoint"
