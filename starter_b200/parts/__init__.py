from .attention import GroupedQueryAttention
from .base import ROLES, ParamSpec, Part, Role, register_role, role_of
from .block import PreNormBlock
from .feedforward import GatedFeedForward
from .norm import RMSNorm
from .registry import FAMILIES, lookup, register
from .rotary import Rotation, RotaryTable

__all__ = ["FAMILIES", "ROLES", "Role", "register_role", "role_of", "GatedFeedForward", "GroupedQueryAttention", "ParamSpec", "Part",
           "PreNormBlock", "RMSNorm", "RotaryTable", "Rotation", "lookup", "register"]
