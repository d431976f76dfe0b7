from .base import (BatchShape, Block, FeedForward, KVCacheView, KVPages, Mixer, Norm, NormSink, ParamSpec, Part, PlanView,
                   PositionEncoding, RowScaled, Runtime, StateCacheView, StateSlot, StepContext, StepPlan)
from .attention import GQAttention
from .block import ParallelBlock, PreNormBlock
from .causal_taps import CausalTaps
from .gated_recurrence import GatedLinearRecurrence
from .latent_attention import LatentAttention
from .embedding import OutputHead, TokenEmbedding
from .linear import Linear
from .mlp import GatedFeedForward, SwiGLUFeedForward
from .norm import GroupRMSNorm, RMSNorm
from .rope import RotaryEmbedding

__all__ = [
    "BatchShape", "Block", "FeedForward", "KVCacheView", "KVPages", "Mixer", "Norm", "NormSink", "ParamSpec", "Part", "PlanView",
    "PositionEncoding", "RowScaled", "Runtime", "StateCacheView", "StateSlot", "StepContext", "StepPlan", "GQAttention", "PreNormBlock", "OutputHead",
    "TokenEmbedding", "Linear", "SwiGLUFeedForward", "RMSNorm", "RotaryEmbedding", "ParallelBlock", "CausalTaps",
    "GatedLinearRecurrence", "LatentAttention", "GatedFeedForward", "GroupRMSNorm",
]
