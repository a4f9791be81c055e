"""The parts layers are made of.  Importing this package registers the
built-in kinds; more can be added with
:func:`inferflux_b200.config.registry.register_part`."""
from .base import Part, KVNeed, StateNeed, RunInfo
from .linear import Linear
from .norm import LayerNorm, RMSNorm
from .position import RotaryHalf
from .attention import GQAttention
from .feed_forward import PolyNormFF, SwiGLU
from .block import JunctionBlock, ParallelBlock, PreNormBlock
from .embedding import SinusoidNormEmbedding, TokenEmbedding, LinearHead
from .shift import TokenShift
from .recurrent import MinGRU
from .latent_attention import LatentAttention
from .junction import LoopEntry
from .window_attention import WindowAttention
from .retention import Retention
from .side_by_side import SideBySide
from .state_space import Mamba2
from .delta_rule import GeneralDelta
from .gated_linear_attention import GatedLinearAttention

__all__ = ["Part", "KVNeed", "StateNeed", "RunInfo", "Linear", "RMSNorm", "RotaryHalf",
           "GQAttention", "SwiGLU", "PreNormBlock", "TokenEmbedding", "LinearHead", "LayerNorm", "PolyNormFF",
           "ParallelBlock", "JunctionBlock", "SinusoidNormEmbedding", "TokenShift", "MinGRU", "LatentAttention",
           "LoopEntry"]
