"""The single-token step captured in CUDA graphs, one per batch size and length class, self-feeding.

A decode step at small batch is hundreds of short kernels; launched one by one the
host is the bottleneck (engine/engine.py:9-12).  The step for ``B`` sequences reads
everything that changes from fixed device buffers (each row's token, position,
slot, length and sampling settings) so one capture serves every step
(engine/engine.py:805-809, 1029-1059).  The sampling kernel writes the drawn token
back as the row's next input and advances its position, so consecutive steps of an
unchanged batch need no host-to-device traffic at all (engine/engine.py:835-838).
Unlike the reference, lengths are per row, and a batch that shrinks simply uses
the graph of the smaller size.

The graph runs the same model code and kernels as the eager step; it is captured
the first time a batch size is used at a length class (how the attention cuts a
sequence's keys into parts is decided at capture, from the class's shortest length).
"""

from __future__ import annotations

import gc
import weakref

import numpy as np
import torch

from .. import ops
from .batch import StepContext


class DecodeGraphs:
    def __init__(self, runner, max_batch: int):
        # the runner owns this object; a weak reference back keeps the pair out of the cycle
        # collector's hands, so that their pinned buffers are freed when the runner is dropped and
        # not at some later moment of the collector's choosing (for instance in the middle of a
        # stream capture, where freeing pinned memory that a stream has used is not allowed)
        self._runner = weakref.ref(runner)
        self.max_batch = max_batch
        dev = runner.device
        # one int32 buffer holds every per-row field, so one copy refreshes a batch
        self.fields = ("tokens", "tok_pos", "tok_slot", "kv_len", "temperature", "key")
        self.meta = torch.zeros((len(self.fields), max_batch), dtype=torch.int32, device=dev)
        self.rows = torch.arange(max_batch, dtype=torch.int32, device=dev)
        self.ones = torch.ones(max_batch, dtype=torch.int32, device=dev)
        self.zeros = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.out = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        # two pinned staging buffers in turn: a copy may still be reading one when the next is filled
        self._stage = [torch.zeros((len(self.fields), max_batch), dtype=torch.int32).pin_memory() for _ in range(2)]
        self._stage_np = [t.numpy() for t in self._stage]
        self._stage_f32 = [a.view(np.float32) for a in self._stage_np]
        self._stage_u32 = [a.view(np.uint32) for a in self._stage_np]
        self._stage_done = [None, None]
        self._views = {}
        self._stage_next = 0
        # drawn tokens travel to the host through two pinned buffers in turn, so that the next step
        # can be launched before the host has looked at this one's tokens (engine/engine.py:1081-1099)
        self._out_host = [torch.zeros((max_batch,), dtype=torch.int32).pin_memory() for _ in range(2)]
        self._out_done = [torch.cuda.Event(), torch.cuda.Event()]
        self._out_next = 0
        self.graphs = {}
        self.logits = {}   # per graph, the float32 logits [batch, vocab] its last replay left
        self.last_key = None  # the graph that ran last
        self.kernels_per_replay = {}  # this library's kernels inside each graph
        self.fed = None  # the slots whose next inputs the device already holds
        self.fed_lengths = None  # and the lengths (tokens in the cache) the device holds them at
        self.kv_hint = 0  # the length the graph being captured is sized for (splits of the attention)

    @property
    def runner(self):
        runner = self._runner()
        if runner is None:
            raise RuntimeError("the runner these graphs belong to is gone")
        return runner

    def _field(self, name, batch):
        return self.meta[self.fields.index(name), :batch]

    def context(self, batch: int) -> StepContext:
        return StepContext(
            n_tokens=batch, n_seqs=batch,
            tokens=self._field("tokens", batch), tok_pos=self._field("tok_pos", batch),
            tok_slot=self._field("tok_slot", batch), seq_slot=self._field("tok_slot", batch),
            seq_q_start=self.rows[:batch], seq_q_len=self.ones[:batch],
            seq_kv_len=self._field("kv_len", batch), want_rows=self.rows[:batch],
            tile_seq=self.rows[:batch], tile_first=self.zeros[:batch],
            block_seq=self.rows[:batch], block_first=self.zeros[:batch],
            max_q_len=1, max_kv_len=self.kv_hint, cache=self.runner.cache, status=self.runner.status,
            host=None)

    def _body(self, batch: int):
        model = self.runner.model
        ctx = self.context(batch)
        logits = model.forward(ctx, ctx.want_rows)
        ops.sample(logits, self._field("temperature", batch).view(torch.float32),
                   self._field("key", batch), self._field("kv_len", batch),
                   status=self.runner.status, out=self.out[:batch],
                   feed=(self._field("tokens", batch), self._field("tok_pos", batch),
                         self._field("kv_len", batch)))
        return logits

    def drop(self) -> None:
        """Forget every captured graph (device tables they read were reallocated)."""
        self.graphs.clear()
        self.logits.clear()
        self.kernels_per_replay.clear()

    def _capture(self, batch: int, key) -> None:
        # nothing may be freed behind the capture's back: collect what is collectable now and keep
        # the cycle collector out until the graph is made
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            self._capture_now(batch, key)
        finally:
            if collecting:
                gc.enable()

    def _capture_now(self, batch: int, key) -> None:
        # tables that grow with the sequence are sized for the longest sequence the cache can hold
        # before anything is captured, so that a long generation does not move them mid-way
        cache = self.runner.cache
        self.runner.model.prepare(cache.max_pages_per_sequence * ops.PAGE_TOKENS)
        saved = self.meta.clone()
        # warm up on a side stream (compiles kernels, sizes library workspaces), then capture;
        # both run the real step on the live sequences.  What the step changes is put back
        # afterwards: the fields, and the fixed-size state of every mixer that keeps one (a running
        # sum would otherwise be advanced by the warm-up).  Keys and values need no care: the warm-up
        # writes this step's own rows, which the real step writes again before they are ever read.
        saved_state = {entry: tensor.clone() for entry, tensor in cache.state.items()}
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.meta.copy_(saved)
                self._body(batch)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.meta.copy_(saved)
        for entry, tensor in saved_state.items():
            cache.state[entry].copy_(tensor)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph):
            self.logits[key] = self._body(batch)
        self.kernels_per_replay[batch] = ops.launch_count - before
        self.graphs[key] = graph
        self.meta.copy_(saved)
        for entry, tensor in saved_state.items():
            cache.state[entry].copy_(tensor)
        torch.cuda.synchronize()

    def load(self, slots, tokens, positions, temperatures, keys) -> None:
        """Put a batch's rows on the device (one copy).  ``tokens`` None: the device keeps the tokens
        it drew itself and only the fields the host owns are refreshed."""
        batch = len(slots)
        turn = self._stage_next
        self._stage_next = 1 - turn
        done = self._stage_done[turn]
        if done is None:
            done = self._stage_done[turn] = torch.cuda.Event()
        else:
            done.synchronize()            # the copy that last read this buffer has long finished
        host = self._stage_np[turn]
        first = 0 if tokens is not None else 1
        if tokens is not None:
            host[0, :batch] = tokens
        host[1, :batch] = positions
        host[2, :batch] = slots
        host[3, :batch] = host[1, :batch] + 1
        self._stage_f32[turn][4, :batch] = temperatures
        self._stage_u32[turn][5, :batch] = keys
        views = self._views.get((turn, batch, first))
        if views is None:
            views = self._views[(turn, batch, first)] = (self.meta[first:, :batch],
                                                          self._stage[turn][first:, :batch])
        views[0].copy_(views[1], non_blocking=True)
        done.record()
        self.fed = tuple(slots)
        self.fed_lengths = list(positions)

    def replay(self, batch: int, kv_tokens: int = 0) -> torch.Tensor:
        """Run one step for the ``batch`` rows on the device; returns the drawn tokens (device).

        ``kv_tokens`` is the longest sequence of the batch (this step's token included).  How the
        attention cuts the keys into parts is fixed when a graph is captured, so there is a graph
        per batch size and per length class (``hint_pages``); a class's graph assumes the class's
        shortest length, which keeps every part at a page or more for all lengths of the class."""
        pages = hint_pages(kv_tokens)
        key = (batch, pages)
        if key not in self.graphs:
            self.kv_hint = pages * ops.PAGE_TOKENS
            self._capture(batch, key)
        self.graphs[key].replay()
        self.last_key = key
        return self.out[:batch]

    def fetch(self, batch: int) -> DrawnTokens:
        """Start the copy of the last replay's tokens to pinned host memory; nothing waits here."""
        turn = self._out_next
        self._out_next = 1 - turn
        self._out_host[turn][:batch].copy_(self.out[:batch], non_blocking=True)
        self._out_done[turn].record()
        return DrawnTokens(self._out_host[turn], self._out_done[turn], batch)


class DrawnTokens:
    """The tokens of a step that is (or was) running: ``result()`` waits for them and returns a list."""

    def __init__(self, host=None, done=None, batch=0, ready=None):
        self._host, self._done, self._batch, self._ready = host, done, batch, ready
        #: True if the device also kept these tokens as the sequences' next inputs, so that the next
        #: step can be launched without them
        self.device_feeds = ready is None

    def result(self) -> list:
        if self._ready is None:
            self._done.synchronize()
            self._ready = self._host[:self._batch].tolist()
        return self._ready


#: length classes of the captured decode graphs, in cache pages: powers of two and their 1.5-folds
HINT_PAGES = tuple(sorted({p for e in range(16) for p in (1 << e, 3 << e >> 1) if p >= 1}))


def hint_pages(kv_tokens: int) -> int:
    """The largest class of ``HINT_PAGES`` that is not longer than ``kv_tokens`` tokens (at least 1)."""
    pages = max(1, -(-kv_tokens // ops.PAGE_TOKENS))
    best = 1
    for p in HINT_PAGES:
        if p <= pages:
            best = p
    return best
