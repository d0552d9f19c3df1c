from .base import (BuildContext, ParamSpec, Part, PartSpec, ProductChoice, build_part,
                   known_parts, register_part, unregister_part)
from .block import Block, PreNormBlock
from .feedforward import FeedForward, SwiGLU
from .io import Embedding, Head, LinearHead, TokenEmbedding
from .linear import Linear
from .mixer import GQAAttention, Mixer
from .norm import Norm, RMSNorm, residual_add
from .plan import LayerPlan, ModelPlan, ScheduleEntry
from .position import NoPosition, PositionEncoding, RotaryHalfSplit, RotaryTable

__all__ = ["BuildContext", "ParamSpec", "Part", "PartSpec", "ProductChoice", "build_part", "known_parts",
           "register_part", "unregister_part", "Block", "PreNormBlock", "FeedForward", "SwiGLU",
           "Embedding", "Head", "LinearHead", "TokenEmbedding", "Linear", "GQAAttention", "Mixer",
           "Norm", "RMSNorm", "residual_add", "LayerPlan", "ModelPlan", "ScheduleEntry",
           "NoPosition", "PositionEncoding", "RotaryHalfSplit", "RotaryTable"]
