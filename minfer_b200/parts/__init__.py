"""The parts that ship with the library, registered under their kinds."""
from ..registry import register_part
from .attention import Attention
from .base import (Block, CacheRequest, CacheView, CallBinding, FeedForward, Mixer, Norm, Part,
                   PositionEncoding, StateRequest, StepContext)
from .block import OutputNormBlock, PreNormBlock, TokenSide
from .delta_rule import GatedDeltaRule
from .latent_attention import LatentAttention
from .linear import Linear
from .mamba2 import Mamba2
from .mlp import DenseMlp, GatedMlp
from .moe import RoutedExperts
from .norm import RmsNorm
from .parallel import ParallelMixer
from .positions import LearnedPositions
from .qknorm_attention import QkNormAttention
from .retention import Retention
from .rotary import NoPosition, Rotary
from .selective_scan import SelectiveScan
from .shift import TokenShift
from .sink_attention import SinkAttention
from .talking_attention import TalkingAttention
from .stream import DepthAverage, EmbeddingNorm, LogitSoftcap, PassInjection

register_part("norm", "rms_norm", RmsNorm, replace=True)
register_part("position", "rotary", Rotary, replace=True)
register_part("position", "none", NoPosition, replace=True)
register_part("mixer", "attention", Attention, replace=True)
register_part("mixer", "sink_attention", SinkAttention, replace=True)
register_part("mixer", "qk_norm_attention", QkNormAttention, replace=True)
register_part("mixer", "latent_attention", LatentAttention, replace=True)
register_part("mixer", "mamba2", Mamba2, replace=True)
register_part("mixer", "gated_delta_rule", GatedDeltaRule, replace=True)
register_part("mixer", "talking_attention", TalkingAttention, replace=True)
register_part("mixer", "retention", Retention, replace=True)
register_part("mixer", "selective_scan", SelectiveScan, replace=True)
register_part("mixer", "parallel", ParallelMixer, replace=True)
register_part("feed_forward", "gated_mlp", GatedMlp, replace=True)
register_part("feed_forward", "dense_mlp", DenseMlp, replace=True)
register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
register_part("model", "learned_positions", LearnedPositions, replace=True)
register_part("model", "embedding_norm", EmbeddingNorm, replace=True)
register_part("model", "logit_softcap", LogitSoftcap, replace=True)
register_part("model", "pass_injection", PassInjection, replace=True)
register_part("model", "depth_average", DepthAverage, replace=True)
register_part("block", "pre_norm", lambda layer, **options: PreNormBlock(layer, **options),
              replace=True)
register_part("block", "output_norm", lambda layer, **options: OutputNormBlock(layer, **options),
              replace=True)
