from .bsms import BistrideMultiLayerGraph, BistrideMultiLayerGraphDataset, bistride_select
from .hydrographnet_dataset import HydroGraphDataset
from .lagrangian_dataset import LagrangianDataset, graph_update
from .mesh_graph_dataset import MeshGraphTimeSeriesDataset, VortexSheddingDataset
from .static_graph_datasets import AhmedBodyDataset, DrivAerNetDataset, StaticMeshGraphDataset, StokesDataset
from .utils import cells_to_edges, edge_features, load_json, save_json

__all__ = ["AhmedBodyDataset", "BistrideMultiLayerGraph", "BistrideMultiLayerGraphDataset", "DrivAerNetDataset", "HydroGraphDataset",
           "LagrangianDataset", "MeshGraphTimeSeriesDataset", "StaticMeshGraphDataset", "StokesDataset", "VortexSheddingDataset",
           "bistride_select", "cells_to_edges", "edge_features", "graph_update", "load_json", "save_json"]
