from .attention import ATTENTION_WORK, AttentionWork, GQAAttention
from .base import (Block, BuildEnv, CacheNeed, FeedForward, KVRequest, LayerCache, Mixer, Norm, Part,
                   PositionEncoding, StateRequest, StepPlanner, TokenFilter)
from .block import DepthAveragedBlock, ParallelBlock, PreNormBlock, SandwichNormBlock
from .conv import CausalShortConv
from .embedding import LMHead, TokenEmbedding
from .latent_attention import LATENT_WORK, LatentAttention, LatentWork
from .linear_attention import DecayLinearAttention, ForgetGateLinearAttention
from .delta_rule import GatedDeltaRule
from .mlp import DenseFF, PolyNormFF, SwiGLU
from .moe import RoutedMoE, TableMoE
from .parallel import ParallelMixers
from .sink_attention import SinkWindowAttention
from .sinusoid import SinusoidalPositions
from .state_space import ScalarDecayStateSpace
from .model import Layer, Model, tensor_specs_of
from .norm import DynamicTanh, RMSNorm
from .normed_attention import NormedGatedAttention
from .registry import (lookup, register, register_block, register_feed_forward, register_mixer,
                       register_norm, register_position_encoding)
from .rope import RotaryEncoding, rotary_inv_freq
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

register("mixer", "gqa_attention", GQAAttention)
register("feed_forward", "swiglu", SwiGLU)
register("norm", "rmsnorm", RMSNorm)
register("position_encoding", "rotary", RotaryEncoding)
register("block", "prenorm", PreNormBlock)
register("embedding", "token_embedding", TokenEmbedding)
register("head", "lm_head", LMHead)
register("mixer", "latent_attention", LatentAttention)
register("mixer", "decay_linear_attention", DecayLinearAttention)
register("feed_forward", "polynorm_ff", PolyNormFF)
register("feed_forward", "table_moe", TableMoE)
register("filter", "causal_short_conv", CausalShortConv)
register("block", "prenorm_depth_average", DepthAveragedBlock)
register("block", "sandwich_norm", SandwichNormBlock)
register("mixer", "parallel_mixers", ParallelMixers)
register("mixer", "scalar_decay_state_space", ScalarDecayStateSpace)
register("feed_forward", "routed_moe", RoutedMoE)
register("mixer", "sink_window_attention", SinkWindowAttention)
register("mixer", "gated_delta_rule", GatedDeltaRule)
register("feed_forward", "dense_ff", DenseFF)
register("position_encoding", "sinusoidal", SinusoidalPositions)
register("norm", "dynamic_tanh", DynamicTanh)
register("block", "parallel_depth_average", ParallelBlock)
register("mixer", "forget_gate_linear_attention", ForgetGateLinearAttention)
register("mixer", "normed_gated_attention", NormedGatedAttention)

__all__ = ["ATTENTION_WORK", "AttentionWork", "GQAAttention", "Block", "BuildEnv", "CacheNeed", "FeedForward",
           "KVRequest", "LayerCache", "Mixer", "Norm", "Part", "PositionEncoding", "StateRequest", "StepPlanner", "PreNormBlock", "LMHead",
           "TokenEmbedding", "SwiGLU", "Layer", "Model", "tensor_specs_of", "RMSNorm", "lookup",
           "register", "register_block", "register_feed_forward", "register_mixer",
           "register_norm", "register_position_encoding", "RotaryEncoding", "rotary_inv_freq",
           "LayerSpec", "ModelSpec", "PartSpec", "RunStep", "TokenFilter", "DepthAveragedBlock", "CausalShortConv",
           "LatentAttention", "DecayLinearAttention", "PolyNormFF", "TableMoE", "SandwichNormBlock", "ParallelMixers",
           "ScalarDecayStateSpace", "RoutedMoE", "SinkWindowAttention", "GatedDeltaRule", "DenseFF", "SinusoidalPositions",
           "DynamicTanh", "ParallelBlock", "ForgetGateLinearAttention", "NormedGatedAttention"]
