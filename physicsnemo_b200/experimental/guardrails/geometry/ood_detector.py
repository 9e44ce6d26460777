"""Geometry guardrail: flags surface meshes whose global shape descriptors are unlikely under the training set.

Counterpart of ``physicsnemo/experimental/guardrails/geometry/ood_detector.py`` (``GeometryGuardrail`` :39).  Fit a
density model on the descriptors of training meshes; a query returns for every mesh the percentile of its anomaly score
among the training scores and a status: ``OK`` below ``warn_pct``, ``WARN`` below ``reject_pct``, ``REJECT`` above.
The fitted guardrail is stored as one ``.npz`` (no pickled objects) together with the descriptor schema, which is
verified on load.  Directory helpers read the ``.npz`` meshes written by ``datapipes.mesh_dataset.save_mesh_npz``
(STL / VTK readers need packages that are import-gated elsewhere in this framework).
"""

from __future__ import annotations

from pathlib import Path
from typing import List, Optional, Union

import numpy as np
import torch

from ....mesh import Mesh
from .density_model import GeometryDensityModel
from .feature_extraction import FEATURE_NAMES, FEATURE_VERSION, FeatureSchema, extract_features, feature_hash

__all__ = ["GeometryGuardrail"]


class GeometryGuardrail:
    def __init__(self, method: str = "gmm", gmm_components: int = 1, pce_components: Optional[int] = None, warn_pct: float = 99.0,
                 reject_pct: float = 99.9, poly_degree: int = 2, interaction_only: bool = False, random_state: Optional[int] = 0,
                 device: Union[str, torch.device] = "cpu"):
        if not 0 <= warn_pct <= reject_pct <= 100:
            raise ValueError(f"need 0 <= warn_pct <= reject_pct <= 100, got {warn_pct} and {reject_pct}")
        self.warn_pct, self.reject_pct, self.device = warn_pct, reject_pct, torch.device(device)
        self.feature_names, self.feature_version, self.feature_hash = FEATURE_NAMES, FEATURE_VERSION, feature_hash(FEATURE_NAMES)
        self.density = GeometryDensityModel(method=method, gmm_components=gmm_components, pce_components=pce_components,
                                            poly_degree=poly_degree, interaction_only=interaction_only, random_state=random_state,
                                            device=self.device)

    def _features(self, meshes: List[Mesh]) -> torch.Tensor:
        X = torch.stack([extract_features(m.to(self.device), return_tensor=True) for m in meshes])
        FeatureSchema.validate_array(X.cpu().numpy())
        return X

    @staticmethod
    def _load_dir(mesh_dir: Path):
        from ....datapipes.mesh_dataset import MeshReader

        files = sorted(Path(mesh_dir).glob("*.npz"))
        reader = MeshReader(files)
        return [reader[i] for i in range(len(files))], [f.stem for f in files]

    def fit(self, meshes: List[Mesh]) -> None:
        if not meshes:
            raise ValueError("Cannot fit on empty list of meshes")
        self.density.fit(self._features(meshes))

    def fit_from_dir(self, mesh_dir: Path) -> None:
        meshes, _ = self._load_dir(mesh_dir)
        if not meshes:
            raise ValueError("No valid features extracted from mesh files")
        self.fit(meshes)

    def _classify(self, pct: float) -> str:
        return "REJECT" if pct >= self.reject_pct else ("WARN" if pct >= self.warn_pct else "OK")

    def query(self, meshes: List[Mesh]) -> List[dict]:
        if not meshes:
            raise ValueError("Cannot query empty list of meshes")
        pcts = self.density.percentiles(self.density.score(self._features(meshes)))
        return [{"percentile": float(p), "status": self._classify(p)} for p in pcts]

    def query_from_dir(self, mesh_dir: Path) -> List[dict]:
        meshes, names = self._load_dir(mesh_dir)
        if not meshes:
            raise ValueError("No valid features extracted from mesh files")
        return [dict(name=n, **r) for n, r in zip(names, self.query(meshes))]

    def save(self, path: Path) -> None:
        if self.density.ref_scores is None:
            raise RuntimeError("Guardrail not fitted. Call fit() before saving.")
        state = {k: v for k, v in self.density.get_state().items() if v is not None}
        np.savez(path, **state, warn_pct=self.warn_pct, reject_pct=self.reject_pct, feature_names=np.array(self.feature_names, dtype="U100"),
                 feature_version=self.feature_version, feature_hash=self.feature_hash)

    @classmethod
    def load(cls, path: Path, device: Union[str, torch.device] = "cpu") -> "GeometryGuardrail":
        data = np.load(path, allow_pickle=False)
        if str(data["feature_version"]) != FEATURE_VERSION:
            raise RuntimeError(f"Feature version mismatch: saved model uses {data['feature_version']}, but current code expects {FEATURE_VERSION}")
        if [str(n) for n in data["feature_names"]] != FEATURE_NAMES:
            raise RuntimeError("Feature schema mismatch: saved model uses different feature names")
        if str(data["feature_hash"]) != feature_hash(FEATURE_NAMES):
            raise RuntimeError("Feature hash mismatch: saved model may have been corrupted or uses a different feature extraction implementation")
        for key in ("method", "ref_scores"):
            if key not in data:
                raise RuntimeError(f"Missing required key '{key}' in saved file")
        guard = cls(method=str(data["method"]), warn_pct=float(data["warn_pct"]), reject_pct=float(data["reject_pct"]), device=device)
        guard.density.set_state({k: data[k] for k in data.files}, device=device)
        return guard
