from .graph_cast_net import GraphCastNet  # noqa: F401
