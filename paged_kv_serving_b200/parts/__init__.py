"""Layer parts: norm, position encoding, mixer, feed-forward, their arrangement in a block, and the
embedding and head at a model's two ends."""

from paged_kv_serving_b200.parts.attention import PagedAttention
from paged_kv_serving_b200.parts.base import (
    Block, CacheBinding, GroupView, IntArena, Normed, PagedKVRequest, ParamSpec, Part, StateRequest, StepContext,
)
from paged_kv_serving_b200.parts.block import ConvSideBlock, PostNormBlock, PreNormBlock, SandwichBlock
from paged_kv_serving_b200.parts.conv import ResidualCausalConv
from paged_kv_serving_b200.parts.feed_forward import BiasedDense, Dense, GatedDense, GatedRoutedExperts, RoutedExperts, SwiGLU
from paged_kv_serving_b200.parts.io import LinearHead, PassInput, TokenEmbedding
from paged_kv_serving_b200.parts.latent_attention import LatentAttention
from paged_kv_serving_b200.parts.lightning import LightningAttention
from paged_kv_serving_b200.parts.linear_attention import GatedLinearAttention, Retention
from paged_kv_serving_b200.parts.mamba import Mamba1
from paged_kv_serving_b200.parts.mlstm import MLSTM
from paged_kv_serving_b200.parts.parallel import ParallelMixers
from paged_kv_serving_b200.parts.norms import IdentityNorm, LayerNorm, OffsetRMSNorm, RMSNorm, ScalarRMSNorm
from paged_kv_serving_b200.parts.position import NoPositionEncoding, PositionEncoding, RotaryEncoding, ScaledRotaryFrequencies
from paged_kv_serving_b200.parts.sink_attention import SinkWindowAttention
from paged_kv_serving_b200.parts.token_shift import TokenShift
from paged_kv_serving_b200.parts.token_side import TokenSideInput, TokenSideTable

__all__ = [
    "GatedDense", "GatedLinearAttention", "ParallelMixers", "PassInput", "Retention",
    "Dense", "LayerNorm", "LightningAttention", "SandwichBlock", "TokenShift",
    "GatedRoutedExperts", "IdentityNorm", "Mamba1", "OffsetRMSNorm", "PostNormBlock", "ScaledRotaryFrequencies", "SinkWindowAttention",
    "BiasedDense", "Block", "CacheBinding", "ConvSideBlock", "GroupView", "IntArena", "LatentAttention", "LinearHead", "MLSTM",
    "NoPositionEncoding", "Normed", "PagedAttention", "PagedKVRequest", "ParamSpec", "Part", "PositionEncoding",
    "PreNormBlock", "RMSNorm", "ResidualCausalConv", "RotaryEncoding", "RoutedExperts", "ScalarRMSNorm", "StateRequest",
    "StepContext", "SwiGLU", "TokenEmbedding", "TokenSideInput", "TokenSideTable",
]
