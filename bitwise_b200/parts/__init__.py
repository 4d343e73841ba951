from .attention import GQAAttention
from .base import (FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, FeedForward, Mixer, Norm, PagedKVNeed,
                   PagedKVView, Part, PositionEncoding, SlotStateNeed, SlotStateView, StepContext, Workspace,
                   register_feed_forward, register_mixer, register_norm, register_position_encoding)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .mlp import SwiGLU
from .norm import RMSNorm
from .rope import RotaryEncoding, inverse_frequencies
