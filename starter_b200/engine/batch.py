"""One step's batch: which tokens run, to which sequence each belongs and where it sits in it.

Tokens of all sequences are packed one after another.  Per token the device gets
its id, its absolute position in its sequence and its sequence's slot; per sequence
the slot, where its tokens start in the packing, how many there are and how long
the sequence is once they are in the cache.  That is all a part needs to treat a
whole prompt, a later chunk of one and a single token alike.  The integers travel
in ONE pinned buffer and one copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


QUERY_TILE = 64
QUERY_BLOCK = 256      # what one block of the tensor-core prompt attention takes

#: in place of a token id in a ``StepEntry``: "the token the device drew for this sequence in the step
#: before" (a captured single-token step can go on from it before the host has seen it)
FED = None


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the places (indices into
    ``tokens``) whose logits are wanted."""

    slot: int
    tokens: list
    want: list = field(default_factory=list)


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor
    tok_pos: torch.Tensor
    tok_slot: torch.Tensor
    seq_slot: torch.Tensor
    seq_q_start: torch.Tensor
    seq_q_len: torch.Tensor
    seq_kv_len: torch.Tensor
    want_rows: torch.Tensor
    tile_seq: torch.Tensor      # work list of the many-token attention: per tile of 64 queries its
    tile_first: torch.Tensor    # sequence (index into the seq_* arrays) and its first query there
    block_seq: torch.Tensor     # the same list in blocks of 256 queries (None: derive it from the tiles)
    block_first: torch.Tensor
    max_q_len: int
    max_kv_len: int
    cache: object
    status: torch.Tensor
    #: the same arrays as numpy on the host, for parts that plan per sequence.  ``None`` in a captured
    #: (CUDA-graph) step: nothing of the host may steer it, so a part that wants to run there works
    #: from the device arrays above alone (every sequence then brings exactly one token, row ``i``
    #: belongs to ``seq_slot[i]``)
    host: dict
    #: True once the step's first kernel has run as an ordinary (not dependent) launch: everything
    #: earlier steps wrote is then complete before any kernel of this step starts, and a kernel may
    #: read it before its own dependent-launch wait.  Set by the model; False for a context made by hand.
    fenced: bool = False

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1


def plan_step(entries, starts, vocab_size=None):
    """Host arithmetic of a step: returns the packed int32 arrays as a dict of numpy arrays.

    ``starts[i]`` is the number of tokens sequence ``i`` already has in the cache.
    """
    if not entries:
        raise ValueError("a step needs at least one sequence")
    slots = [e.slot for e in entries]
    if len(set(slots)) != len(slots):
        raise ValueError("a sequence appears twice in one step")
    tokens, tok_pos, tok_slot, want_rows = [], [], [], []
    q_start, q_len, kv_len = [], [], []
    for entry, start in zip(entries, starts):
        n = len(entry.tokens)
        if n == 0:
            raise ValueError(f"the sequence in slot {entry.slot} brings no token to this step")
        base = len(tokens)
        for w in entry.want:
            if not 0 <= w < n:
                raise ValueError(f"logits wanted at place {w} of a sequence that brings {n} tokens")
            want_rows.append(base + w)
        if vocab_size is not None:
            for t in entry.tokens:
                if not 0 <= t < vocab_size:
                    raise ValueError(f"token id {t} is outside the vocabulary of {vocab_size}")
        tokens.extend(entry.tokens)
        tok_pos.extend(range(start, start + n))
        tok_slot.extend([entry.slot] * n)
        q_start.append(base)
        q_len.append(n)
        kv_len.append(start + n)
    # tiles of 64 queries, the ones with most keys to walk first
    tiles = [(kv_len[i] - q_len[i] + first, i, first)
             for i in range(len(entries)) for first in range(0, q_len[i], QUERY_TILE)]
    tiles.sort(key=lambda t: -t[0])
    blocks = [(kv_len[i] - q_len[i] + first, i, first)
              for i in range(len(entries)) for first in range(0, q_len[i], QUERY_BLOCK)]
    blocks.sort(key=lambda t: -t[0])
    arrays = {
        "tokens": tokens, "tok_pos": tok_pos, "tok_slot": tok_slot, "seq_slot": slots,
        "seq_q_start": q_start, "seq_q_len": q_len, "seq_kv_len": kv_len, "want_rows": want_rows,
        "tile_seq": [t[1] for t in tiles], "tile_first": [t[2] for t in tiles],
        "block_seq": [t[1] for t in blocks], "block_first": [t[2] for t in blocks],
    }
    return {k: np.asarray(v, dtype=np.int32) for k, v in arrays.items()}


def upload(arrays: dict, device) -> dict:
    """Copy the int32 arrays to the device in one transfer; returns tensors that view one buffer."""
    order = list(arrays)
    sizes = [arrays[k].size for k in order]
    # keep every array 16-byte aligned inside the buffer
    offsets, total = [], 0
    for size in sizes:
        offsets.append(total)
        total += (size + 3) // 4 * 4
    host = torch.empty((max(total, 4),), dtype=torch.int32, pin_memory=torch.cuda.is_available())
    view = host.numpy()
    for key, off, size in zip(order, offsets, sizes):
        view[off:off + size] = arrays[key]
    dev = host.to(device, non_blocking=True)
    return {key: dev[off:off + size] for key, off, size in zip(order, offsets, sizes)}
