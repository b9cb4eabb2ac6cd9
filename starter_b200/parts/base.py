"""What every layer part has in common: named parameters with stated shapes, set once after loading.

A part is built from its spec and a working dtype, says which tensors it wants
(``param_specs``), receives them (``set_params``) and then computes.  It never
learns which model it sits in: tensor names in a checkpoint are the layer spec's
business, sizes and constants arrive through the part's own spec.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class ParamSpec:
    """``role`` is ``"matrix"`` (kept in the working dtype) or ``"gain"`` (a norm's scale: kept in the
    working dtype unless the checkpoint stores it in 32-bit, which then stays so)."""

    shape: tuple
    role: str = "matrix"


class Part:
    def __init__(self, spec, dtype):
        self.spec = spec
        self.dtype = dtype

    def param_specs(self) -> dict:
        return {}

    def set_params(self, params: dict) -> None:
        if params:
            raise ValueError(f"{type(self).__name__} takes no parameters")

    def weight_bytes(self) -> int:
        """Bytes of parameters one step reads (for the bandwidth account)."""
        return 0


def bytes_of(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))
