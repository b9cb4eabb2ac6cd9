"""Choosing the next token: greedy, or a draw at a temperature.

The reference is greedy only (``argmax``, engine/engine.py:833, 1077); temperature
sampling is this library's addition.  A draw is ``argmax(logits / t + g)`` with
Gumbel noise ``g``, which is distributed as ``softmax(logits / t)``.  The noise is a
pure function of (sampling seed, request number, position of the drawn token,
vocabulary index), so what a request draws does not depend on its batch.  The
kernel is csrc/sampling.cu; ``gumbel_noise`` states the same arithmetic on the host.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import ops


@dataclass(frozen=True)
class SamplingParams:
    """``temperature`` 0 means greedy."""

    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")


def _mix32(x):
    x = np.asarray(x, dtype=np.uint32).copy()
    x ^= x >> np.uint32(16)
    x *= np.uint32(0x7FEB352D)
    x ^= x >> np.uint32(15)
    x *= np.uint32(0x846CA68B)
    x ^= x >> np.uint32(16)
    return x


def request_key(seed: int, request_number: int) -> int:
    """The 32-bit key of one request's random stream."""
    with np.errstate(over="ignore"):
        return int(_mix32(np.uint32(request_number & 0xFFFFFFFF) + _mix32(np.uint32(seed & 0xFFFFFFFF))))


def gumbel_noise(key: int, position: int, vocab: int) -> np.ndarray:
    """The float32 noise the kernel adds for the token drawn at ``position`` of a request."""
    with np.errstate(over="ignore"):
        row_key = _mix32(np.uint32(position) + _mix32(np.uint32(key)))
        r = _mix32(np.arange(vocab, dtype=np.uint32) ^ row_key)
    u = ((r >> np.uint32(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)


class Sampler:
    """Selects one token per row of device logits; per-row temperature, key and position."""

    def __init__(self, device, status=None):
        self.device = device
        self.status = status

    def select(self, logits, temperatures, keys, positions) -> list:
        """``logits`` float32 ``[B, V]`` on the device; the rest are host lists.  Returns host ints."""
        return self.select_device(logits, temperatures, keys, positions).tolist()

    def select_device(self, logits, temperatures, keys, positions) -> torch.Tensor:
        if all(t <= 0 for t in temperatures):
            return ops.sample(logits, status=self.status)
        meta = np.empty((3, len(temperatures)), dtype=np.int32)
        meta[0] = np.asarray(temperatures, dtype=np.float32).view(np.int32)
        meta[1] = np.asarray(keys, dtype=np.uint32).view(np.int32)
        meta[2] = np.asarray(positions, dtype=np.int32)
        dev = torch.from_numpy(meta).to(self.device, non_blocking=True)
        return ops.sample(logits, dev[0].view(torch.float32), dev[1], dev[2], status=self.status)
