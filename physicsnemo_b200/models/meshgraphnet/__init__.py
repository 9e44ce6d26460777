from .meshgraphnet import MeshGraphNet, MeshGraphNetProcessor
