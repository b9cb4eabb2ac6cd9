"""Rotary position tables: cos and sin of ``position * theta ** (-2j / head_dim)``.

The angles are formed in float32 exactly as the reference forms them
(engine/engine.py:240-259): exponent ``arange(0, D, 2) / D``, ``inv_freq = 1 /
theta ** exponent``, ``outer(position, inv_freq)``.  The two halves of the
reference's ``[positions, D]`` table are equal, so only ``D / 2`` columns are kept.
The tables stay float32; the kernel that applies them rounds to the working type
where the reference casts (before any multiply).  Tables are computed on the host
so that they are the same bits on every machine, and grow on demand.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import Part


@dataclass(frozen=True)
class Rotation:
    """What a mixer needs to rotate queries and keys: float32 tables ``[positions, rotary_dim / 2]``,
    how many leading dimensions of a head they turn, and how the two halves of a pair lie in a head
    (``"half_split"``: element ``j`` with element ``j + rotary_dim / 2``; ``"interleaved"``: ``2j``
    with ``2j + 1``).  The kernels say which of these they take (``ops.rotation_tables``)."""

    cos: torch.Tensor
    sin: torch.Tensor
    rotary_dim: int
    layout: str = "half_split"


class RotaryTable(Part):
    MIN_POSITIONS = 4096

    def __init__(self, spec, dtype, device="cuda"):
        super().__init__(spec, dtype)
        self.device = device
        self.length = 0
        self.cos = None
        self.sin = None

    @staticmethod
    def angles(theta: float, head_dim: int, length: int) -> torch.Tensor:
        exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim
        inv_freq = 1.0 / (theta ** exponent)
        pos = torch.arange(length, dtype=torch.int64).float()
        return torch.outer(pos, inv_freq)

    def rotation(self) -> Rotation:
        """The tables as they are now (call ``ensure`` first): the whole head, half-split."""
        return Rotation(self.cos, self.sin, self.spec.head_dim, "half_split")

    def ensure(self, length: int) -> bool:
        """Make the tables cover positions ``[0, length)``; True if they moved (captured graphs that
        read the old tables must then be dropped)."""
        if length <= self.length:
            return False
        size = max(self.MIN_POSITIONS, self.length)
        while size < length:
            size *= 2
        freqs = self.angles(self.spec.theta, self.spec.head_dim, size)
        self.cos = freqs.cos().contiguous().to(self.device)
        self.sin = freqs.sin().contiguous().to(self.device)
        self.length = size
        return True
