from .base import MATRIX, TABLE, VECTOR, ParamSpec, Part
from .context import Runtime, StepContext
from .norm import LayerNorm, RMSNorm
from .rope import RampRotaryEmbedding, RotaryEmbedding, inverse_frequencies, ramp_frequencies
from .attention import Attention
from .mamba2 import Mamba2
from .mlp import GatedMLP
from .gla import GatedLinearAttention
from .latent_attention import LatentAttention
from .moe import ClampedGLU, DenseMLP, RoutedMLP
from .mingru import MinGRU
from .pooled_attention import PooledWindowAttention
from .delta import ChannelDelta, GatedDelta
from .conv_attention import ConvAttention
from .lightning import LightningAttention
from .sink_attention import MixerPair, SinkAttention
from .moe import GLU
from .embedding import BareLMHead, Embedding, LMHead, NormedEmbedding, PairEmbedding, StreamEmbedding
from .block import ParallelStreamBlock, PostNormBlock, PreNormParallelBlock, PreNormStreamBlock, StreamInput, TokenSideInput, OutNormStreamBlock

__all__ = ["MATRIX", "TABLE", "VECTOR", "ParamSpec", "Part", "Runtime", "StepContext", "RMSNorm",
           "RotaryEmbedding", "inverse_frequencies", "Attention", "Mamba2", "GatedMLP", "Embedding", "LMHead",
           "PreNormParallelBlock", "PostNormBlock", "GatedLinearAttention", "LatentAttention", "DenseMLP", "RoutedMLP",
           "PairEmbedding", "BareLMHead", "LayerNorm", "MinGRU", "PooledWindowAttention", "ClampedGLU", "NormedEmbedding",
           "PreNormStreamBlock", "TokenSideInput", "ChannelDelta", "LightningAttention", "MixerPair", "SinkAttention", "GLU",
           "StreamEmbedding", "ParallelStreamBlock", "StreamInput", "GatedDelta", "ConvAttention", "OutNormStreamBlock",
           "RampRotaryEmbedding", "ramp_frequencies"]
