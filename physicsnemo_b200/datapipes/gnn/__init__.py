from .mesh_graph_dataset import MeshGraphTimeSeriesDataset, VortexSheddingDataset
from .utils import cells_to_edges, edge_features, load_json, save_json

__all__ = ["MeshGraphTimeSeriesDataset", "VortexSheddingDataset", "cells_to_edges", "edge_features", "load_json", "save_json"]
