"""Typed descriptions of a decoder: what each layer is made of and in which order layers run.

These dataclasses are the only thing the engine knows about a model.  An
architecture's config class (for instance ``Qwen3Config``) turns its own
``config.json`` keys into a ``ModelSpec``; the parts, the cache and the step
function are built from the spec and never ask which architecture it came from.

Every spec carries a ``kind`` string.  ``starter_b200.parts.registry`` maps a
kind to the class that implements it, so a new mixer, feed-forward, norm or
position encoding is a new spec dataclass plus one registry entry.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    """Root-mean-square norm with a plain gain (no ``1 + w``)."""

    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Half-split rotary position encoding over the whole head."""

    head_dim: int
    theta: float
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a key/value cache.

    ``window`` is ``None`` for attention over all keys, or the number of most
    recent keys (the query's own included) a query may see.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qk_norm: bool
    qk_norm_eps: float
    position: Optional[RopeSpec]
    window: Optional[int] = None
    kind: str = "attention"


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    """Dense gated feed-forward: ``down(act(gate(x)) * up(x))``."""

    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    kind: str = "gated_dense"


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: named part specs and the arrangement that puts them together.

    ``parts`` maps a part's name inside the layer to its spec.  Which names there are and to which
    family each belongs (mixer, feed_forward, norm ...) is the arrangement's business: the pre-norm
    block wants ``mixer``, ``feed_forward``, ``norm1`` and ``norm2``; an arrangement with a third norm,
    without a feed-forward or with two mixers names its own.  ``names`` maps each part's logical
    parameter name (``"mixer.q"``, ``"norm1.weight"`` ...) to the tensor name in the checkpoint.
    """

    parts: dict
    names: dict
    arrangement: str = "prenorm"

    def __getattr__(self, name):
        # layer.mixer, layer.norm1 ...: the spec of the part of that name
        parts = object.__getattribute__(self, "parts")
        if name in parts:
            return parts[name]
        raise AttributeError(f"this layer has no part named {name!r} (it has: {', '.join(parts)})")


def prenorm_layer(mixer, feed_forward, norm1, norm2, names, arrangement: str = "prenorm") -> LayerSpec:
    """The layer of the pre-norm block: ``x + mixer(norm1(x))``, then ``+ feed_forward(norm2(.))``."""
    return LayerSpec({"mixer": mixer, "feed_forward": feed_forward, "norm1": norm1, "norm2": norm2},
                     names, arrangement)


@dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named by several
    entries; its weights are then shared).  ``cache`` names the cache entry the
    mixer uses; entries that share a number share keys and values.  An entry with
    ``writes_cache=False`` only reads the cache another entry filled.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, run order, final norm and output head."""

    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple
    schedule: tuple
    final_norm: object
    tie_embeddings: bool
    embed_name: str
    final_norm_name: str
    lm_head_name: str
    max_position: int = 0
    extra: dict = field(default_factory=dict)

    def cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)


def default_schedule(num_layers: int) -> tuple:
    """Each layer once, in order, each with a cache entry of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(num_layers))
