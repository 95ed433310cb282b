from .base import (TensorSpec, PagedKV, FixedState, StepContext, GroupView,
                   CacheHandle, ResidualStream, Part, Norm, Mixer, FeedForward,
                   PositionEncoding)
from .norm import RMSNorm
from .position import RotaryPosition, rotary_tables
from .attention import GroupedQueryAttention
from .feedforward import SwiGLUFeedForward
from .block import PreNormBlock
from .model import ComposedModel, LayerCall, TokenEmbedding, OutputHead
