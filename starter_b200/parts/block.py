"""How a layer's parts are arranged around the residual stream.

``PreNormBlock``: ``x1 = x + mixer(norm1(x))``, ``x2 = x1 + feed_forward(norm2(x1))``
(engine/engine.py:665-736).  Every residual sum is followed at once by a norm, so
the two are one kernel: a block takes ``(residual, pending)``, where ``pending``
is the previous block's output not yet added, and returns the same pair
(engine/engine.py:669-673).  The model's final norm closes the chain the same way.
A block does not know its neighbours or the model it is in.

A mixer or feed-forward that sets ``adds_to_stream = True`` is called with ``add_to=residual``: it
may add its output onto that tensor itself (in the epilogue of its last product) and return
``ops.ADDED`` instead of the output; the norm that follows then only norms.

An arrangement says which parts it is made of: ``FAMILIES`` maps each part's name inside the layer
to the family its spec is looked up in.  The model builds exactly those parts from the layer spec
and hands them over by name; ``mixer`` names the part that owns the layer's cache entry.
"""

from __future__ import annotations


class PreNormBlock:
    FAMILIES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm"}

    def __init__(self, parts: dict):
        self._parts = dict(parts)
        self.mixer = parts["mixer"]
        self.feed_forward = parts["feed_forward"]
        self.norm1 = parts["norm1"]
        self.norm2 = parts["norm2"]

    def parts(self) -> dict:
        return dict(self._parts)

    def __call__(self, residual, pending, ctx, entry, writes_cache=True):
        n = self.norm1.add(residual, pending)
        if getattr(self.mixer, "adds_to_stream", False):
            a = self.mixer(n, ctx, entry, writes_cache, add_to=residual)
        else:
            a = self.mixer(n, ctx, entry, writes_cache)
        m = self.norm2.add(residual, a)
        if getattr(self.feed_forward, "adds_to_stream", False):
            return residual, self.feed_forward(m, ctx, add_to=residual)
        return residual, self.feed_forward(m, ctx)
