"""The cache: one slot per live sequence, paged keys and values per cache entry, per-sequence state.

Memory is a pool of pages of 64 tokens.  A sequence owns a slot (a row of the
block table) and as many pages as its length needs; ``block_table[slot][i]`` is
the page that holds its tokens ``64 * i .. 64 * i + 63``.  Every cache entry of a
group stores that page at the same index of its own tensor, so one table serves
all entries.  Groups (entries with the same heads, head size and window) have
storage of their own.  Next to the pages sits fixed-size state per slot for
mixers that ask for it; it is zeroed when a sequence opens.

The reference keeps ``[batch, kv_heads, capacity, head_dim]`` per layer and one
position for the whole batch (engine/engine.py:856-871); here each sequence has
its own length, and only positions below it are ever read, so stale contents of
reused pages are harmless (the invariant of engine/engine.py:1075-1076, per slot).
"""

from __future__ import annotations

import numpy as np
import torch

from .allocator import CacheFull, IndexAllocator
from .layout import PAGE_TOKENS, KVNeed, StateNeed, pages_for, plan_groups

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class SequenceCache:
    """``kv_needs``/``state_needs`` map a cache entry number to its ``KVNeed``/``StateNeed``."""

    def __init__(self, kv_needs: dict, state_needs: dict, max_tokens: int, max_sequences: int,
                 dtype, device, max_sequence_tokens: int | None = None):
        if max_tokens <= 0 or max_sequences <= 0:
            raise ValueError("the cache needs room for at least one token and one sequence")
        self.dtype = dtype
        self.device = torch.device(device)
        self.num_pages = pages_for(max_tokens)
        self.max_sequences = max_sequences
        per_seq = self.num_pages if max_sequence_tokens is None else min(
            self.num_pages, pages_for(max_sequence_tokens))
        self.max_pages_per_sequence = per_seq
        self.slots = IndexAllocator(max_sequences, "slot")
        self.pages = IndexAllocator(self.num_pages, "page")
        self.lengths = [0] * max_sequences
        self._owned = [[] for _ in range(max_sequences)]
        self._table_host = np.zeros((max_sequences, per_seq), dtype=np.int32)
        self.block_table = torch.zeros((max_sequences, per_seq), dtype=torch.int32, device=self.device)
        self._dirty = {}  # slot -> (first, last+1) columns of the table not yet on the device
        # changed table entries travel through pinned staging memory, two buffers in turn, so that
        # the copies need not block and a buffer is not refilled while a copy may still read it
        pin = self.device.type == "cuda"
        self._stage = [torch.zeros((max_sequences * per_seq,), dtype=torch.int32, pin_memory=pin)
                       for _ in range(2)]
        self._stage_done = [None, None]
        self._stage_next = 0

        self.groups = plan_groups(kv_needs)
        self._where = {}
        self.keys, self.values = [], []
        for g, group in enumerate(self.groups):
            need: KVNeed = group.need
            shape = (len(group.entries), self.num_pages, need.num_kv_heads, PAGE_TOKENS, need.head_dim)
            self.keys.append(torch.zeros(shape, dtype=dtype, device=self.device))
            self.values.append(torch.zeros(shape, dtype=dtype, device=self.device))
            for i, entry in enumerate(group.entries):
                self._where[entry] = (g, i)
        self.state = {}
        for entry, need in state_needs.items():
            if need is None:
                continue
            need: StateNeed
            self.state[entry] = torch.zeros((max_sequences,) + tuple(need.shape),
                                            dtype=_STATE_DTYPES[need.dtype], device=self.device)

    # ------------------------------------------------------------------ storage views

    def entry_pages(self, entry: int):
        """``(keys, values)`` of one cache entry, each ``[pages, kv_heads, 64, head_dim]``."""
        g, i = self._where[entry]
        return self.keys[g][i], self.values[g][i]

    def entry_need(self, entry: int) -> KVNeed:
        return self.groups[self._where[entry][0]].need

    def entry_state(self, entry: int):
        return self.state.get(entry)

    def bytes_per_token(self) -> int:
        total = 0
        for group in self.groups:
            total += 2 * len(group.entries) * group.need.num_kv_heads * group.need.head_dim * self.dtype.itemsize
        return total

    # ------------------------------------------------------------------ sequences

    def open_sequence(self) -> int:
        """A free slot with length 0, no pages, and zeroed state."""
        slot = self.slots.take()
        self.lengths[slot] = 0
        self._owned[slot] = []
        for tensor in self.state.values():
            tensor[slot].zero_()
        return slot

    def reserve(self, slot: int, length: int) -> None:
        """Make sure ``slot`` owns pages for ``length`` tokens (its length itself does not change)."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not open")
        have = len(self._owned[slot])
        want = pages_for(length)
        if want <= have:
            return
        if want > self.max_pages_per_sequence:
            raise CacheFull(f"a sequence of {length} tokens needs {want} pages; the table holds "
                            f"{self.max_pages_per_sequence} per sequence")
        fresh = self.pages.take_many(want - have)
        self._owned[slot].extend(fresh)
        self._table_host[slot, have:want] = fresh
        first, last = self._dirty.get(slot, (have, want))
        self._dirty[slot] = (min(first, have), max(last, want))

    def advance(self, slot: int, tokens: int) -> int:
        """Record that ``tokens`` more tokens of ``slot`` are (being) written; returns the old length."""
        old = self.lengths[slot]
        new = old + tokens
        if pages_for(new) > len(self._owned[slot]):
            raise CacheFull(f"slot {slot} holds pages for {len(self._owned[slot]) * PAGE_TOKENS} "
                            f"tokens, {new} needed; reserve first")
        self.lengths[slot] = new
        return old

    def close_sequence(self, slot: int) -> None:
        """Give back the slot and its pages."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not open, so it cannot be closed")
        for page in self._owned[slot]:
            self.pages.give_back(page)
        self._owned[slot] = []
        self.lengths[slot] = 0
        self._dirty.pop(slot, None)
        self.slots.give_back(slot)

    def owned_pages(self, slot: int) -> list:
        return list(self._owned[slot])

    def sync_table(self) -> None:
        """Copy block-table entries that changed since the last call to the device (asynchronously,
        in stream order: kernels launched after this call see them)."""
        if not self._dirty:
            return
        turn = self._stage_next
        self._stage_next = 1 - turn
        stage = self._stage[turn]
        if self.device.type == "cuda":
            done = self._stage_done[turn]
            if done is None:
                done = self._stage_done[turn] = torch.cuda.Event()
            else:
                done.synchronize()        # the copies that last read this buffer have long finished
        at = 0
        view = stage.numpy()
        for slot, (first, last) in self._dirty.items():
            n = last - first
            view[at:at + n] = self._table_host[slot, first:last]
            self.block_table[slot, first:last].copy_(stage[at:at + n], non_blocking=True)
            at += n
        if self.device.type == "cuda":
            done.record()
        self._dirty.clear()

    def check(self) -> None:
        """No slot or page lost, held twice, or owned by two sequences."""
        self.slots.check()
        self.pages.check()
        seen = set()
        for slot in range(self.max_sequences):
            owned = self._owned[slot]
            if owned and not self.slots.is_held(slot):
                raise AssertionError(f"closed slot {slot} still owns pages")
            for page in owned:
                if page in seen:
                    raise AssertionError(f"page {page} is owned twice")
                if not self.pages.is_held(page):
                    raise AssertionError(f"page {page} is owned by slot {slot} but marked free")
                seen.add(page)
        if len(seen) != self.pages.held_count:
            raise AssertionError("a held page belongs to no sequence")
