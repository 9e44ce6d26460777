"""HealDA building blocks: packed observation context and the temporal / pixel-observation attention layers."""

from .adaln import AdaLNModulation, gated_residual, modulate
from .attention_layers import CrossAttentionModuleBase, PixelCrossAttention, TemporalAttention, mask_causal
from .healda import HealDA
from .video_dit import VideoDiT, VideoDiTBlock
from .video_healda import VideoHealDA
from .obs_tokenizer import ObsTokenizerFiLM
from .sharding import shard_t, shard_t_shardtensor, shard_x, shard_x_shardtensor
from .point_embed import MultiSensorObsEmbedder, ObsTokenizer, SensorEmbedder, UniformFusion
from .scatter_aggregator import ScatterAggregator, scatter_mean
from .obs_context import (ObsContext, PixelGroupMap, build_pixel_group_map, counts_to_cu_seqlens, prepare_obs_context,
                          sort_and_pack)

__all__ = ["HealDA", "VideoDiT", "VideoDiTBlock", "VideoHealDA", "AdaLNModulation", "gated_residual", "modulate", "CrossAttentionModuleBase", "ObsContext", "ObsTokenizerFiLM", "ScatterAggregator", "scatter_mean", "MultiSensorObsEmbedder", "ObsTokenizer", "SensorEmbedder", "UniformFusion", "shard_t", "shard_t_shardtensor", "shard_x", "shard_x_shardtensor", "PixelCrossAttention", "PixelGroupMap", "TemporalAttention",
           "build_pixel_group_map", "counts_to_cu_seqlens", "mask_causal", "prepare_obs_context", "sort_and_pack"]
