"""Ball query layer (parity: ``physicsnemo/nn/module/ball_query.py``): for every grid point the (up to)
``neighbors_in_radius`` cloud points within ``radius`` — or the reverse — through the ``radius_search``
functional (cell-list CUDA kernels on GPU)."""
import torch
import torch.nn as nn

from ..functional.neighbors import radius_search


class BQWarp(nn.Module):
    def __init__(self, radius: float = 0.25, neighbors_in_radius: int | None = 10):
        super().__init__()
        self.radius, self.neighbors_in_radius = radius, neighbors_in_radius

    def forward(self, x: torch.Tensor, p_grid: torch.Tensor, reverse_mapping: bool = True):
        if p_grid.shape[-1] != x.shape[-1] or x.shape[-1] != 3:
            raise ValueError("The last dimension of p_grid and x must be 3")
        if p_grid.ndim in (4, 5):
            p_grid = p_grid.reshape(p_grid.shape[0], -1, 3)
        elif p_grid.ndim != 3:
            raise ValueError("p_grid must be 3D, 4D, 5D only")
        points, queries = (x, p_grid) if reverse_mapping else (p_grid, x)
        mapping, outputs = radius_search(points, queries, self.radius, self.neighbors_in_radius, return_points=True)
        return mapping, outputs
