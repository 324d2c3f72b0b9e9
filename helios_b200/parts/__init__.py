from .base import (Block, DeferredNorm, FeedForward, InputStage, LayerCache, Mixer, Norm, OutputStage, PagedCacheSpec, Part,
                   PositionEncoding, StateSpec, WeightSpec, known_parts, part_class,
                   register_part)
from .norm import RMSNorm
from .rotary import RotaryEncoding, rotary_frequencies
from .attention import GQAAttention
from .mlp import SwiGLU
from .embedding import NormedHead, OutputHead, TokenEmbedding
from .block import PreNormBlock
from .plan import ModelPlan, Run

__all__ = ["Block", "DeferredNorm", "FeedForward", "InputStage", "OutputStage", "NormedHead", "LayerCache", "Mixer", "Norm", "PagedCacheSpec", "Part",
           "PositionEncoding", "StateSpec", "WeightSpec", "known_parts", "part_class",
           "register_part", "RMSNorm", "RotaryEncoding", "rotary_frequencies", "GQAAttention",
           "SwiGLU", "OutputHead", "TokenEmbedding", "PreNormBlock", "ModelPlan", "Run"]
