"""Model parts: each owns its sizes, constants and parameters, none knows its model."""
from .base import (FeedForward, KVCacheSpec, Mixer, Norm, Param, Part, PlanView, PositionEncoding, Segments,
                   StateSpec, StepContext, StepPlanner)
from .linear import Linear, StackedLinear
from .norm import ExactRMSNorm, LayerNorm, RMSNorm
from .rotary import RotaryEmbedding, RotaryFrequencies, rotary_table
from .attention import GroupedQueryAttention
from .feed_forward import GatedMLP, PlainMLP
from .experts import RoutedExperts
from .linear_attention import DecayLinearAttention, GatedLinearAttention
from .latent_attention import LatentAttention
from .parallel import ParallelMixers
from .block import PostNormBlock, PreNormBlock, SandwichNormBlock
from .side_input import TokenSideInput
from .decoder import DecoderModel, LayerCall, TokenEmbedding
