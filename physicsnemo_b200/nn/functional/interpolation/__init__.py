from .interpolation import (GridToPointInterpolation, PointToGridInterpolation, grid_to_point_interpolation,
                            interpolation, point_to_grid_interpolation)
