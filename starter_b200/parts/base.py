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
class Role:
    """What a kind of tensor is drawn from in the random-weights mode (``mean``, ``std``) and how it is
    placed on the device: ``keep_32bit`` tensors that the checkpoint stores in 32-bit stay so (the
    others are cast to the working type)."""

    mean: float
    std: float
    keep_32bit: bool = False


#: the roles a parameter can have.  ``matrix``: a projection, N(0, 0.02), working type.  ``gain``: a
#: norm's scale, 1 + N(0, 0.1).  ``bias``: an additive term, N(0, 0.02).  ``state``: a per-channel
#: constant of a recurrence (a decay, a time step, a short convolution), N(0, 0.1), kept in 32-bit when
#: stored so.  A part with another kind of tensor registers its role; an unknown role is an error,
#: never silently a matrix.
ROLES = {
    "matrix": Role(0.0, 0.02),
    "gain": Role(1.0, 0.1, keep_32bit=True),
    "bias": Role(0.0, 0.02, keep_32bit=True),
    "state": Role(0.0, 0.1, keep_32bit=True),
}


def register_role(name: str, role: Role) -> None:
    ROLES[name] = role


def role_of(name: str) -> Role:
    try:
        return ROLES[name]
    except KeyError:
        raise ValueError(f"no tensor role {name!r} is registered (known: {', '.join(sorted(ROLES))})") from None


@dataclass(frozen=True)
class ParamSpec:
    """A parameter's shape and its ``role`` (see ``ROLES``)."""

    shape: tuple
    role: str = "matrix"

    def __post_init__(self):
        role_of(self.role)


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
