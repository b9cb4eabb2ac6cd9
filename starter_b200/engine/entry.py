"""The Python entry point, in the reference's manner: ``Engine(model_path).generate(input_ids,
max_new_tokens)`` yields one list of token ids per step (README.md:54-66, engine/engine.py:1069-1105).

Kept from the reference: the names and meanings of ``model_path``, ``input_ids`` and
``max_new_tokens``; exactly ``max_new_tokens`` yields of one id per sequence, in
the order the sequences arrived; greedy; an end-of-sequence id is an ordinary id.
Added: sequences of one call may differ in length; ``dtype`` picks the bfloat16
serving path or the true float32 path; ``complete`` is the library-level call with
temperature, seeds, stop tokens, early finish and several batches.
"""

from __future__ import annotations

import torch

from ..cache.layout import PAGE_TOKENS
from ..sampling.sampler import Sampler, SamplingParams
from .generate import Completion, GenerationLoop, Request, pages_held
from .runner import ModelRunner, load_model


class Engine:
    def __init__(self, model_path: str, dtype: str = "bfloat16", max_batch: int = 64,
                 max_tokens: int | None = None, device: str = "cuda:0") -> None:
        """Load the model in ``model_path`` (``config.json`` + safetensors).  ``max_tokens`` sizes the
        cache (tokens over all live sequences, in cache pages); by default it is sized by the first
        call that needs it and grown by a later call that needs more."""
        self.model = load_model(model_path, dtype, device)
        self.max_batch = max_batch
        self.runner = None
        self._fixed_tokens = max_tokens
        if max_tokens is not None:
            self._build_runner(max_tokens)
        print(f"[engine] loaded {len(self.model.blocks)} layers as {self.model.dtype}", flush=True)

    @classmethod
    def from_model(cls, model, max_batch: int = 64, max_tokens: int | None = None) -> "Engine":
        """An engine around a model that is already on the device (for instance random weights)."""
        self = cls.__new__(cls)
        self.model = model
        self.max_batch = max_batch
        self.runner = None
        self._fixed_tokens = max_tokens
        if max_tokens is not None:
            self._build_runner(max_tokens)
        return self

    def _build_runner(self, max_tokens: int, longest: int | None = None) -> None:
        self.runner = None
        torch.cuda.empty_cache()
        self.runner = ModelRunner(self.model, max_tokens, max_sequences=max(self.max_batch, 1),
                                  max_sequence_tokens=longest)
        self.sampler = Sampler(self.model.device, self.runner.status)

    def _ensure_room(self, requests, batch: int) -> GenerationLoop:
        pages = sorted((pages_held(r) for r in requests), reverse=True)
        need = sum(pages[:batch]) * PAGE_TOKENS
        cache = self.runner.cache if self.runner is not None else None
        small = cache is not None and self._fixed_tokens is None and (
            need > cache.num_pages * PAGE_TOKENS or pages[0] > cache.max_pages_per_sequence)
        if cache is None or small:
            print(f"[engine] building the cache for {need} tokens", flush=True)
            self._build_runner(max(need, PAGE_TOKENS), None if self._fixed_tokens else pages[0] * PAGE_TOKENS)
        return GenerationLoop(self.runner, self.sampler, batch, self.runner.cache.num_pages)

    # ------------------------------------------------------------------ the reference's call

    @torch.inference_mode()
    def generate(self, input_ids: list, max_new_tokens: int):
        """Greedy continuation of every sequence, one step at a time: yields, ``max_new_tokens``
        times, a list with one token id per sequence.  Never stops at an end-of-sequence id."""
        requests = [Request(list(ids), max_new_tokens) for ids in input_ids]
        if max_new_tokens <= 0 or not requests:
            return
        if len(requests) > self.max_batch:
            self.max_batch = len(requests)
            self.runner = None
        loop = self._ensure_room(requests, len(requests))
        for step_out in loop.stream_batch(requests):
            yield [step_out[i] for i in range(len(requests))]

    # ------------------------------------------------------------------ the library-level call

    @torch.inference_mode()
    def complete(self, input_ids: list, max_new_tokens, temperature: float = 0.0, seed: int = 0,
                 stop_token_ids=()) -> list:
        """Generate for every prompt; returns a ``Completion`` (tokens, finish reason) per prompt.

        ``max_new_tokens`` is one number or one per prompt.  Prompts run in batches of at most
        ``max_batch``, one batch after another; a sequence ends at a stop token (kept as its last
        token) or at its length."""
        if isinstance(max_new_tokens, int):
            max_new_tokens = [max_new_tokens] * len(input_ids)
        sampling = SamplingParams(temperature=temperature, seed=seed)
        requests = [Request(list(ids), n, sampling, frozenset(stop_token_ids), number=i)
                    for i, (ids, n) in enumerate(zip(input_ids, max_new_tokens))]
        if not requests:
            return []
        loop = self._ensure_room(requests, min(self.max_batch, len(requests)))
        out = loop.run(requests)
        self.runner.check_status()
        return out


__all__ = ["Completion", "Engine", "Request", "SamplingParams"]
