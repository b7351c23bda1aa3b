from .base import Part, Runtime, build_part, register_part
from .linear import gated_linear, linear
from . import norm, position, attention, mlp, block, embedding, latent_attention, channel_delta, routed_experts, capped_attention, table_experts, state_space, side_by_side, token_side  # noqa: F401  (registers the built-in parts)
from .attention import Attention
from .capped_attention import CappedAttention
from .channel_delta import ChannelDelta
from .latent_attention import LatentAttention
from .routed_experts import RoutedExperts
from .embedding import OutputHead, TokenEmbedding
from .block import ParallelBlock, PreNormBlock, Reinject, SandwichBlock, ScaledParallelBlock
from .mlp import ClampedGatedMLP, GatedMLP, PlainMLP, PolyNormMLP
from .side_by_side import SideBySideMixers
from .state_space import StateSpace
from .token_side import TokenSideInput
from .table_experts import TableExperts
from .norm import RMSNorm
from .position import NoPosition, Rotary

__all__ = ["Part", "Runtime", "build_part", "register_part", "linear", "gated_linear", "Attention", "PreNormBlock",
           "GatedMLP", "PlainMLP", "PolyNormMLP", "ClampedGatedMLP", "SandwichBlock", "ParallelBlock", "ScaledParallelBlock", "SideBySideMixers", "StateSpace", "TokenSideInput", "Reinject", "CappedAttention", "TableExperts", "LatentAttention", "ChannelDelta", "RoutedExperts", "RMSNorm", "NoPosition", "Rotary", "TokenEmbedding", "OutputHead"]
