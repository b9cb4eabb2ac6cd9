"""From a spec's ``kind`` to the class that implements it.

To add a part: write a spec dataclass with a new ``kind``, a class with the
interface of its family (see the existing ones), and register it here or from
your own module with ``register``.  Nothing else in the library changes.

Families and their interfaces
  mixer         ``__init__(spec, dtype, position)``; ``param_specs()``, ``set_params(params)``,
                ``kv_need()`` -> ``KVNeed`` or None, ``state_need()`` -> ``StateNeed`` or None,
                ``prepare(max_position)``, ``__call__(x, ctx, entry, writes_cache)`` -> ``[T, H]``
  feed_forward  ``__init__(spec, dtype)``; ``param_specs()``, ``set_params``, ``__call__(x, ctx)``
  norm          ``__init__(spec, dtype)``; ``param_specs()``, ``set_params``, ``__call__(x)``,
                ``add(residual, delta)``, ``add_rows(residual, delta, rows)``
  position      ``__init__(spec, dtype, device)``; ``ensure(length)`` -> True if device tables moved;
                ``rotation()`` -> ``Rotation`` (tables, how many dimensions of a head they turn and
                in which layout) for mixers that rotate queries and keys
  arrangement   class attribute ``FAMILIES`` (part name -> family); ``__init__(parts: dict)``;
                ``parts()``; attribute ``mixer`` (the part that owns the layer's cache entry);
                ``__call__(residual, pending, ctx, entry, writes_cache)`` -> ``(residual, pending)``
"""

from __future__ import annotations

from .attention import GroupedQueryAttention
from .block import PreNormBlock
from .feedforward import GatedFeedForward
from .norm import RMSNorm
from .rotary import RotaryTable

FAMILIES = ("mixer", "feed_forward", "norm", "position", "arrangement")
_REGISTRY = {family: {} for family in FAMILIES}


def register(family: str, kind: str, cls) -> None:
    if family not in _REGISTRY:
        raise ValueError(f"unknown part family {family!r}; families: {', '.join(FAMILIES)}")
    _REGISTRY[family][kind] = cls


def lookup(family: str, kind: str):
    try:
        return _REGISTRY[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(family, {}))) or "none"
        raise ValueError(f"no {family} of kind {kind!r} is registered (known: {known})") from None


register("mixer", "attention", GroupedQueryAttention)
register("feed_forward", "gated_dense", GatedFeedForward)
register("norm", "rmsnorm", RMSNorm)
register("position", "rope", RotaryTable)
register("arrangement", "prenorm", PreNormBlock)
