from .attention import GatedPagedAttention, PagedAttention, plan_attention_tiles
from .base import (Block, FeedForward, KVNeed, LayerCache, Mixer, Norm, Part, PositionEncoding, PostNormed, ProjectedMixer, Rows, RowSum, Runtime, Scaled, StateNeed,
                   StepContext, StepShape, Workspace, as_rows, known_parts, make_part, register_part)
from .block import EmbeddingReentryBlock, HyperConnectionBlock, PreNormBlock, ReinjectionBlock, SandwichNormBlock, ScaledPreNormBlock
from .conv import ResidualShortConv
from .decoder import CachePlan, DecoderModel, LayerRun
from .delta_rule import GatedDeltaRule
from .feedforward import DenseBiasedMLP, DenseSwiGLU, GroupLimitedGLUExperts, RoutedExperts, SoftmaxRoutedMLPExperts
from .latent_attention import LatentAttention, rotary_frequencies
from .linear_attention import GatedLinearAttention, RetentionMixer, TimeMixWKV
from .linear import grouped_linear, grouped_swiglu_linear, interleave_gate_up, linear, swiglu_linear
from .parallel import ParallelMixers
from .norms import GroupRMSNorm, RMSNorm, StreamRMSNorm, add_to_residual
from .recurrent import HGRN2, InputConvMixer
from .positions import (InterleavedRope, NoPositionWithTemperature, UnfusedEncoding, llama3_scaled_frequencies,
                        wavelength_scaled_frequencies, yarn_frequencies)

__all__ = [
    "EmbeddingReentryBlock", "GatedDeltaRule", "wavelength_scaled_frequencies", "yarn_frequencies", "HyperConnectionBlock",
    "GroupLimitedGLUExperts", "RetentionMixer", "StreamRMSNorm",
    "GatedLinearAttention", "GatedPagedAttention", "ParallelMixers", "ProjectedMixer", "Scaled", "ScaledPreNormBlock",
    "SoftmaxRoutedMLPExperts", "TimeMixWKV",
    "DenseBiasedMLP", "GroupRMSNorm", "HGRN2", "InputConvMixer", "LatentAttention", "PostNormed", "ReinjectionBlock",
    "ResidualShortConv", "SandwichNormBlock", "add_to_residual", "rotary_frequencies",
    "Block", "CachePlan", "DecoderModel", "DenseSwiGLU", "FeedForward", "InterleavedRope", "KVNeed", "LayerCache",
    "LayerRun", "Mixer", "NoPositionWithTemperature", "Norm", "PagedAttention", "Part", "PositionEncoding",
    "PreNormBlock", "RMSNorm", "RoutedExperts", "Rows", "RowSum", "Runtime", "Workspace", "as_rows", "grouped_swiglu_linear", "interleave_gate_up", "swiglu_linear", "StateNeed", "StepContext", "StepShape", "plan_attention_tiles", "UnfusedEncoding",
    "grouped_linear", "known_parts", "linear", "llama3_scaled_frequencies", "make_part", "register_part",
]
