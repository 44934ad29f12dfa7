"""Parts a layer is put together from, and their registration."""
from ..registry import register_part
from .attention import GQAAttention
from .base import Block, BuildContext, CacheSpec, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import PreNormBlock
from .branches import NormedBranchesMixer
from .embedding import Embedding, Head, LMHead, PositionalTokenEmbedding, SinusoidalTokenEmbedding, TokenEmbedding
from .gated_block import GatedPostNormBlock
from .hyper_block import HyperStreamsBlock
from .latent_attention import LatentAttention
from .mamba2 import Mamba2Mixer
from .matrix_rnn import DecayedLinearMixer, DeltaRuleMixer, GatedLinearMixer, RetentionMixer
from .mlp import DenseMLP, GatedMLP, SwiGLUMLP
from .moe import RoutedExperts
from .sandwich_block import SandwichNormBlock
from .parallel_block import LoopReentry, ParallelBlock, PendingSum
from .window_attention import ConvWindowAttention, RotaryWindowAttention
from .norm import RMSNorm
from .rope import RotaryEmbedding

register_part("norm", "rmsnorm", RMSNorm)
register_part("position", "rope", RotaryEmbedding)
register_part("mixer", "gqa_attention", GQAAttention)
register_part("feed_forward", "swiglu", SwiGLUMLP)
register_part("block", "prenorm", PreNormBlock)
register_part("mixer", "conv_window_attention", ConvWindowAttention)
register_part("feed_forward", "dense", DenseMLP)
register_part("block", "gated_postnorm", GatedPostNormBlock)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "sinusoidal_token_embedding", SinusoidalTokenEmbedding)
register_part("head", "lm_head", LMHead)
register_part("embedding", "positional_token_embedding", PositionalTokenEmbedding)
register_part("mixer", "mamba2", Mamba2Mixer)
register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("mixer", "latent_attention", LatentAttention)
register_part("mixer", "delta_rule", DeltaRuleMixer)
register_part("mixer", "gated_linear", GatedLinearMixer)
register_part("block", "hyper_streams", HyperStreamsBlock)
register_part("mixer", "rotary_window_attention", RotaryWindowAttention)
register_part("mixer", "decayed_linear", DecayedLinearMixer)
register_part("mixer", "retention", RetentionMixer)
register_part("mixer", "normed_branches", NormedBranchesMixer)
register_part("block", "parallel", ParallelBlock)
register_part("reentry", "loop_reentry", LoopReentry)

__all__ = ["Block", "BuildContext", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
           "PreNormBlock", "Embedding", "Head", "LMHead", "TokenEmbedding", "SwiGLUMLP", "DenseMLP", "GatedPostNormBlock",
           "ConvWindowAttention", "SinusoidalTokenEmbedding", "PositionalTokenEmbedding",
           "RotaryWindowAttention", "DecayedLinearMixer", "RetentionMixer", "NormedBranchesMixer", "ParallelBlock", "PendingSum", "LoopReentry",
           "Mamba2Mixer", "LatentAttention", "DeltaRuleMixer", "GatedLinearMixer", "HyperStreamsBlock", "GatedMLP", "RoutedExperts", "SandwichNormBlock", "RMSNorm", "RotaryEmbedding", "GQAAttention"]
