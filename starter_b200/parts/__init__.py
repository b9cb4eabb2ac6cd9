from .attention import GroupedQueryAttention
from .base import ParamSpec, Part
from .block import PreNormBlock
from .feedforward import GatedFeedForward
from .norm import RMSNorm
from .registry import FAMILIES, lookup, register
from .rotary import RotaryTable

__all__ = ["FAMILIES", "GatedFeedForward", "GroupedQueryAttention", "ParamSpec", "Part",
           "PreNormBlock", "RMSNorm", "RotaryTable", "lookup", "register"]
