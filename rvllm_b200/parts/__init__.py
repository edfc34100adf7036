from .base import (Part, TensorSpec, KvCacheNeed, StateNeed, Registry, MIXERS, FEED_FORWARDS, NORMS,
                   POSITION_ENCODINGS, BLOCKS, HOOKS, FAMILIES)
from .linear import Linear
from .norm import RMSNorm
from .rope import RotaryEncoding, inverse_frequencies
from .attention import PagedAttention
from .mlp import GatedMLP
from .block import PreNormResidualBlock, OutputNormResidualBlock, SandwichNormResidualBlock
from .sink_attention import GatedSinkAttention
from .mamba2 import Mamba2Mixer
from .latent_attention import LatentAttention
from .moe import PolyNormMLP, TableMoE
from .hooks import LogitSoftcap, StreamOffset
