"""RMSNorm with a plain gain, alone or fused with the residual sum that always precedes it."""

from __future__ import annotations

from .. import ops
from .base import ParamSpec, Part, bytes_of


class RMSNorm(Part):
    """``y = gain * round(x * rsqrt(mean(x^2) + eps))``; reduce and scale in float
    (engine/engine.py:75-88, engine/kernels/rmsnorm.py:21-45)."""

    def param_specs(self):
        return {"weight": ParamSpec((self.spec.size,), "gain")}

    def set_params(self, params):
        self.weight = params["weight"]

    def __call__(self, x):
        return ops.rmsnorm(x, self.weight, self.spec.eps)

    def add(self, residual, delta):
        """``residual += delta`` in place, then the norm of the sum (engine/kernels/fused.py:115-144)."""
        if delta is None or delta is ops.ADDED:      # nothing open, or the part before added it itself
            return ops.rmsnorm(residual, self.weight, self.spec.eps)
        return ops.rmsnorm(residual, self.weight, self.spec.eps, delta=delta)

    def add_rows(self, residual, delta, rows):
        """The norm of ``(residual + delta)[rows]`` without touching ``residual``."""
        if delta is ops.ADDED:
            delta = None
        return ops.rmsnorm(residual, self.weight, self.spec.eps, delta=delta, rows=rows)

    def weight_bytes(self):
        return bytes_of(self.weight)
