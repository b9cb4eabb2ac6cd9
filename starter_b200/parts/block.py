"""How a layer's parts are arranged around the residual stream.

``PreNormBlock``: ``x1 = x + mixer(norm1(x))``, ``x2 = x1 + feed_forward(norm2(x1))``
(engine/engine.py:665-736).  Every residual sum is followed at once by a norm, so
the two are one kernel: a block takes ``(residual, pending)``, where ``pending``
is the previous block's output not yet added, and returns the same pair
(engine/engine.py:669-673).  The model's final norm closes the chain the same way.
A block does not know its neighbours or the model it is in.
"""

from __future__ import annotations


class PreNormBlock:
    def __init__(self, mixer, feed_forward, norm1, norm2):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norm1 = norm1
        self.norm2 = norm2

    def parts(self) -> dict:
        return {"mixer": self.mixer, "feed_forward": self.feed_forward,
                "norm1": self.norm1, "norm2": self.norm2}

    def __call__(self, residual, pending, ctx, entry, writes_cache=True):
        n = self.norm1.add(residual, pending)
        a = self.mixer(n, ctx, entry, writes_cache)
        m = self.norm2.add(residual, a)
        return residual, self.feed_forward(m, ctx)
