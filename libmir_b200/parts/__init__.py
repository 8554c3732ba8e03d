"""Built-in parts and their registration by kind."""

from ..registry import register_part
from .attention import SoftmaxAttention
from .base import Block, BuildEnv, FeedForward, Mixer, Norm, Part, PartContext, Position, ScratchContext
from .block import ARRANGEMENTS, OutputNormBlock, ParallelBlock, PreNormBlock, StreamMix, StreamsBlock, build_block
from .delta_rule import GatedDeltaRule
from .experts import RoutedExperts
from .feed_forward import GeluMlp, SwiGlu
from .latent_attention import LatentAttention
from .retention import Retention
from .wkv import Wkv
from .side_by_side import SideBySide
from .norm import LayerNorm, RmsNorm
from .rope import Rotary, inverse_frequencies

register_part("rms_norm", RmsNorm)
register_part("layer_norm", LayerNorm)
register_part("stream_mix", StreamMix)
register_part("rotary", Rotary)
register_part("softmax_attention", SoftmaxAttention)
register_part("swiglu", SwiGlu)
register_part("gelu_mlp", GeluMlp)
register_part("gated_delta_rule", GatedDeltaRule)
register_part("side_by_side", SideBySide)
register_part("latent_attention", LatentAttention)
register_part("wkv", Wkv)
register_part("retention", Retention)
register_part("routed_experts", RoutedExperts)

__all__ = ["ARRANGEMENTS", "Block", "BuildEnv", "FeedForward", "GatedDeltaRule", "GeluMlp", "LatentAttention", "LayerNorm", "Mixer", "Norm",
           "OutputNormBlock", "ParallelBlock", "Part", "PartContext", "Position", "PreNormBlock", "Retention", "RmsNorm", "Rotary", "RoutedExperts",
           "ScratchContext", "SideBySide", "SoftmaxAttention", "StreamMix", "StreamsBlock", "SwiGlu", "Wkv", "build_block", "inverse_frequencies"]
