"""AeroJEPA (parity: ``physicsnemo/experimental/models/aerojepa/__init__.py``)."""
from .aerojepa import AeroJEPA, AeroJEPATrunk
from .decoder import QueryTokenDecoder, SirenHead
from .encoders import (BaseContextEncoder, BaseTargetEncoder, ContextTransformer, PointClusterGraphPool, PointTransformer,
                       TargetTransformer, build_geometry_features)
from .predictor import PrototypeTokenJEPAHead
from .tokens import EncoderOutput, TokenSet, pad_token_sets, trim_batched_tokens

__all__ = ["AeroJEPA", "AeroJEPATrunk", "QueryTokenDecoder", "SirenHead", "BaseContextEncoder", "BaseTargetEncoder",
           "ContextTransformer", "TargetTransformer", "PointTransformer", "PointClusterGraphPool", "build_geometry_features",
           "PrototypeTokenJEPAHead", "TokenSet", "EncoderOutput", "pad_token_sets", "trim_batched_tokens"]
