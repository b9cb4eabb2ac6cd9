"""What a model needs from the cache, worked out from its spec before any memory is touched.

Each schedule entry's mixer states its needs: growing per-token keys and values
(``KVNeed``) and/or a fixed-size per-sequence state (``StateNeed``).  Cache entries
with the same needs form a group with storage of its own.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


#: tokens per cache page: the one definition; the kernels' own constant is checked against it when
#: the first kernel library is loaded
PAGE_TOKENS = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass(frozen=True)
class KVNeed:
    """Keys and values per token: ``num_kv_heads * head_dim`` each; ``window`` None = keep all."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per sequence, zero when the sequence starts."""

    shape: tuple
    dtype: str = "float32"


@dataclass
class CacheGroup:
    need: KVNeed
    entries: list  # cache entry numbers, in order; position in this list = index into the storage


def plan_groups(entry_needs: dict) -> list:
    """Group cache entries (``{entry: KVNeed}``) by equal need, keeping entry order."""
    groups = {}
    for entry in sorted(entry_needs):
        need = entry_needs[entry]
        if need is None:
            continue
        groups.setdefault(need, CacheGroup(need=need, entries=[])).entries.append(entry)
    return list(groups.values())
