"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early, and as
many batches one after another as the requests need.

A batch is a set of requests that start together: their prompts run in ONE step,
then every live sequence runs one token per step.  A sequence that draws a stop
token or reaches its ``max_new_tokens`` leaves the batch at once and gives its slot
and pages back; the others go on, and nothing they compute depends on who left.
The reference's loop (engine/engine.py:1069-1105) is the special case of one batch,
equal lengths, greedy, no stop tokens: its contract (exactly ``max_new_tokens``
tokens per sequence, the first from the prompt's logits, the last never fed back)
is kept.

The loop only decides; it talks to a runner (``open_sequence``, ``reserve``,
``step``, ``close_sequence``) and a sampler (``select``), so its decisions can be
tested without a device.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..cache.layout import PAGE_TOKENS, pages_for
from ..sampling.sampler import SamplingParams, request_key
from .batch import FED, StepEntry


@dataclass
class Request:
    prompt: list
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_token_ids: frozenset = frozenset()
    number: int | None = None  # which random stream it draws from; default: its index in the call

    def __post_init__(self):
        if len(self.prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")
        self.stop_token_ids = frozenset(self.stop_token_ids)


@dataclass
class Completion:
    tokens: list
    finish_reason: str  # "stop" (a stop token was drawn; it is the last token) or "length"


class _Ready:
    """The handle of a step whose tokens are already on the host."""

    device_feeds = False      # the device does not hold the next inputs: they go in from the host

    def __init__(self, drawn):
        self._drawn = list(drawn)

    def result(self) -> list:
        return self._drawn


def tokens_held(request: Request) -> int:
    """Cache tokens a request can come to hold: the last drawn token is never fed back."""
    return len(request.prompt) + max(request.max_new_tokens - 1, 0)


def pages_held(request: Request) -> int:
    return pages_for(tokens_held(request))


def plan_batches(requests, max_batch: int, max_pages: int) -> list:
    """Split request indices, in order, into batches of at most ``max_batch`` sequences whose pages
    fit ``max_pages`` together.  Requests that generate nothing are in no batch."""
    if max_batch <= 0:
        raise ValueError("max_batch must be positive")
    batches, current, used = [], [], 0
    for i, req in enumerate(requests):
        if req.max_new_tokens == 0:
            continue
        need = pages_held(req)
        if need > max_pages:
            raise ValueError(f"request {i} needs {need} pages of {PAGE_TOKENS} tokens; the cache has {max_pages}")
        if current and (len(current) == max_batch or used + need > max_pages):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
    return batches


class GenerationLoop:
    def __init__(self, runner, sampler, max_batch: int, max_pages: int, lookahead: bool = True):
        self.runner = runner
        self.sampler = sampler
        self.max_batch = max_batch
        self.max_pages = max_pages
        #: launch a step before the step before it has handed its tokens to the host, where that is
        #: possible (see ``stream_batch``); the tokens are the same either way
        self.lookahead = lookahead

    def _start(self, entries, requests, active, keys, lengths):
        """Launch one step for the ``active`` requests; returns a handle with ``result()``."""
        runner = self.runner
        temps = [requests[i].sampling.temperature for i in active]
        now_keys = [keys[i] for i in active]
        places = [lengths[i] for i in active]
        if hasattr(runner, "start_step"):
            return runner.start_step(entries, self.sampler, temps, now_keys, places)
        if hasattr(runner, "step_and_select"):
            drawn = runner.step_and_select(entries, self.sampler, temps, now_keys, places)
        else:
            drawn = self.sampler.select(runner.step(entries), temps, now_keys, places)
        if hasattr(drawn, "tolist"):
            drawn = drawn.tolist()        # one copy from the device, not one per sequence
        return _Ready(drawn)

    def stream_batch(self, requests, numbers=None):
        """Run one batch; after every step yield ``{position in requests: token}`` for the sequences
        that drew a token in it.  Returns (via ``StopIteration.value``) the list of ``Completion``."""
        runner = self.runner
        n = len(requests)
        numbers = list(numbers) if numbers is not None else [
            r.number if r.number is not None else i for i, r in enumerate(requests)]
        keys = [request_key(r.sampling.seed, num) for r, num in zip(requests, numbers)]
        outputs = [[] for _ in range(n)]
        reasons = [None] * n
        slots = {}
        try:
            active = [i for i, r in enumerate(requests) if r.max_new_tokens > 0]
            for i in range(n):
                if i not in active:
                    reasons[i] = "length"
            for i in active:
                slots[i] = runner.open_sequence()
                runner.reserve(slots[i], tokens_held(requests[i]))
            lengths = {i: len(requests[i].prompt) for i in active}
            entries = [StepEntry(slots[i], list(requests[i].prompt), [len(requests[i].prompt) - 1])
                       for i in active]
            handle = self._start(entries, requests, active, keys, lengths)
            while active:
                # One step of lookahead (engine/engine.py:1081-1099).  Who is in the next step is
                # known before this step's tokens are whenever no live request can stop on a token
                # and none reaches its length now; the device holds the tokens it drew, so the next
                # step is launched first and this step's tokens are read while it runs.
                ahead = None
                if self.lookahead and getattr(handle, "device_feeds", False) and all(
                        not requests[i].stop_token_ids and len(outputs[i]) + 2 <= requests[i].max_new_tokens
                        for i in active):
                    for i in active:
                        lengths[i] += 1
                    ahead = self._start([StepEntry(slots[i], [FED], [0]) for i in active],
                                        requests, active, keys, lengths)
                    for i in active:
                        lengths[i] -= 1
                drawn = handle.result()
                step_out = {}
                still = []
                for i, tok in zip(active, drawn):
                    tok = int(tok)
                    outputs[i].append(tok)
                    step_out[i] = tok
                    lengths[i] += 1
                    if tok in requests[i].stop_token_ids:
                        reasons[i] = "stop"
                    elif len(outputs[i]) >= requests[i].max_new_tokens:
                        reasons[i] = "length"
                    if reasons[i] is None:
                        still.append(i)
                    else:
                        runner.close_sequence(slots.pop(i))
                yield step_out
                active = still
                if ahead is not None:
                    handle = ahead
                elif active:
                    handle = self._start([StepEntry(slots[i], [outputs[i][-1]], [0]) for i in active],
                                         requests, active, keys, lengths)
        finally:
            for slot in slots.values():
                runner.close_sequence(slot)
        return [Completion(outputs[i], reasons[i] or "length") for i in range(n)]

    def run_batch(self, requests, numbers=None) -> list:
        gen = self.stream_batch(requests, numbers)
        while True:
            try:
                next(gen)
            except StopIteration as stop:
                return stop.value

    def run(self, requests) -> list:
        """All requests, as many batches one after another as it takes; results in request order."""
        requests = list(requests)
        results = [Completion([], "length") for _ in requests]
        for batch in plan_batches(requests, self.max_batch, self.max_pages):
            numbers = [requests[i].number if requests[i].number is not None else i for i in batch]
            for i, done in zip(batch, self.run_batch([requests[i] for i in batch], numbers)):
                results[i] = done
        return results
