"""Dense gated feed-forward: ``down(round(silu(gate(x))) * up(x))``, no biases, no routing."""

from __future__ import annotations

import torch

from .. import ops
from .base import ParamSpec, Part, bytes_of


class GatedFeedForward(Part):
    """gate and up are stored stacked as one ``[2 * I, H]`` matrix so one product feeds both
    (engine/engine.py:163, 464-468, 735)."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.activation != "silu":
            raise ValueError(f"the gated feed-forward kernel implements silu, not {spec.activation!r}")

    def param_specs(self):
        h, i = self.spec.hidden_size, self.spec.intermediate_size
        return {"gate": ParamSpec((i, h)), "up": ParamSpec((i, h)), "down": ParamSpec((h, i))}

    def set_params(self, params):
        self.gate_up = torch.cat([params["gate"], params["up"]], dim=0).contiguous()
        self.down = params["down"].contiguous()

    adds_to_stream = True

    def __call__(self, x, ctx=None, add_to=None):
        status = ctx.status if ctx is not None else None
        act = ops.linear(x, self.gate_up, gated=True, status=status)
        return ops.linear(act, self.down, status=status, add_to=add_to)

    def weight_bytes(self):
        return bytes_of(self.gate_up, self.down)
