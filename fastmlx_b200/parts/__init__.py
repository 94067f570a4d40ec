from .attention import GQAAttention
from .base import (FeedForward, Mixer, Norm, PagedKVSpec, Part, PositionEncoding, Run, Runtime,
                   StateSpec, StreamEncoding, WeightSpec)
from .block import MixerOnly, PairMixer, ParallelBlock, PreNormBlock, SandwichBlock
from .delta import GatedDeltaMixer
from .embedding import BigramEmbedding, Embedding, LMHead
from .linear import JoinedLinear, Linear
from .mlp import DenseMLP, SwiGLU
from .model import Model
from .latent import LatentAttention
from .loop import LoopInput, LoopPass
from .moe import PlainRoutedExperts, RoutedExperts
from .retention import RetentionMixer
from .norm import DynamicTanh, Pending, RMSNorm
from .ssm import StateSpaceMixer
from .rope import NoPositionEncoding, RotaryEmbedding, inverse_frequencies

__all__ = ["GQAAttention", "FeedForward", "Mixer", "Norm", "PagedKVSpec", "Part", "PositionEncoding",
           "Run", "Runtime", "StateSpec", "StreamEncoding", "WeightSpec", "PreNormBlock", "Embedding", "LMHead", "Linear",
           "SwiGLU", "DenseMLP", "JoinedLinear", "ParallelBlock", "GatedDeltaMixer", "Model", "RMSNorm", "NoPositionEncoding", "RotaryEmbedding", "inverse_frequencies", "SandwichBlock", "LatentAttention", "LoopInput", "LoopPass", "RoutedExperts",
           "DynamicTanh", "Pending", "BigramEmbedding", "StateSpaceMixer", "PairMixer", "PlainRoutedExperts",
           "RetentionMixer", "MixerOnly"]
