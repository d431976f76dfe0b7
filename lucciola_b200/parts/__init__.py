from .base import (BatchShape, Block, FeedForward, KVCacheView, KVPages, Mixer, Norm, NormSink, ParamSpec, Part, PlanView,
                   PositionEncoding, RowScaled, Runtime, StateCacheView, StateSlot, StepContext, StepPlan)
from .attention import GatedBiasAttention, GQAttention, distance_slopes
from .block import ParallelBlock, PostNormBlock, PreNormBlock
from .causal_taps import CausalTaps
from .decay_attention import DecayLinearAttention
from .experts import RoutedExperts
from .side_by_side import SideBySideMixer
from .gated_recurrence import GatedLinearRecurrence
from .latent_attention import LatentAttention
from .embedding import OutputHead, TokenEmbedding
from .linear import Linear
from .mlp import GatedFeedForward, SwiGLUFeedForward
from .norm import GroupRMSNorm, LayerNorm, RMSNorm
from .rope import RotaryEmbedding

__all__ = [
    "BatchShape", "Block", "FeedForward", "KVCacheView", "KVPages", "Mixer", "Norm", "NormSink", "ParamSpec", "Part", "PlanView",
    "PositionEncoding", "RowScaled", "Runtime", "StateCacheView", "StateSlot", "StepContext", "StepPlan", "GQAttention", "PreNormBlock", "OutputHead",
    "TokenEmbedding", "Linear", "SwiGLUFeedForward", "RMSNorm", "RotaryEmbedding", "ParallelBlock", "CausalTaps",
    "GatedLinearRecurrence", "LatentAttention", "GatedFeedForward", "GroupRMSNorm", "GatedBiasAttention", "distance_slopes",
    "PostNormBlock", "DecayLinearAttention", "RoutedExperts", "SideBySideMixer", "LayerNorm",
]
