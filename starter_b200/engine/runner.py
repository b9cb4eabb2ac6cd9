"""The step function: runs exactly the tokens it is given, as one batch, from the cache.

``ModelRunner`` owns a loaded model and its cache.  ``step`` takes, for each
sequence of the batch, its slot, its next tokens and the places whose logits are
wanted, writes those tokens' keys and values behind what the sequence already
holds, and returns float32 logits ``[wanted, vocab]`` in the order of the entries
and of their ``want`` lists.  A whole prompt, a later chunk of one and a single
token are the same call; sequences of a step may bring different numbers of
tokens.  (The reference has two functions for this, ``_forward_prefill`` and
``_forward_decode``, engine/engine.py:738-839, and needs equal lengths.)
"""

from __future__ import annotations

import os

import torch

from ..cache import SequenceCache, pages_for
from ..config import load_config
from ..weights import load_checkpoint
from .batch import FED, StepContext, StepEntry, plan_step, upload
from .graphs import DecodeGraphs, DrawnTokens
from .model import DecoderModel

DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32,
}


def resolve_dtype(dtype):
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, not {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, not {dtype!r}") from None


def require_cuda(device="cuda:0") -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("starter_b200 runs on a CUDA device (sm_100a); none is visible and there is "
                           "no CPU implementation")
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"starter_b200 runs on CUDA devices only, not {device}")
    torch.cuda.set_device(device)
    # no reduced-precision matrix modes anywhere (engine/engine.py:119-122)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    return device


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """Build the model ``model_dir/config.json`` names and load its safetensors weights."""
    device = require_cuda(device)
    dtype = resolve_dtype(dtype)
    config = load_config(model_dir)
    spec = config.to_model_spec()
    model = DecoderModel(spec, dtype, device)
    alias = (spec.lm_head_name, spec.embed_name) if spec.tie_embeddings else None
    tensors = load_checkpoint(model_dir, model.expected_tensors(), dtype, device, tied_alias=alias)
    model.load_tensors(tensors)
    model.config = config
    return model


def random_model(config, seed: int, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """The model of ``config`` (a typed config) with random weights drawn on the device: no disk.
    (Values differ from a model folder written with the same seed, which is drawn on the CPU.)"""
    from ..weights import random_checkpoint

    device = require_cuda(device)
    dtype = resolve_dtype(dtype)
    model = DecoderModel(config.to_model_spec(), dtype, device)
    model.load_tensors(random_checkpoint(model.expected_tensors(), seed, dtype, device))
    model.config = config
    return model


class ModelRunner:
    def __init__(self, model: DecoderModel, max_tokens: int, max_sequences: int | None = None,
                 max_sequence_tokens: int | None = None, use_graphs: bool = True):
        self.model = model
        self.device = model.device
        pages = pages_for(max_tokens)
        if max_sequences is None:
            max_sequences = min(pages, 1024)
        self.cache = SequenceCache(model.kv_needs(), model.state_needs(), max_tokens, max_sequences,
                                   model.dtype, self.device, max_sequence_tokens)
        self.status = torch.zeros((1,), dtype=torch.int32, device=self.device)
        self.graphs = DecodeGraphs(self, max_sequences) if use_graphs else None
        #: with False, every one-token step gets its inputs from pinned host memory (one small copy
        #: per step: positions, slots, lengths, sampling settings, and the tokens too when the host
        #: has them) instead of going on from what the device holds
        self.self_feeding = True

    # ------------------------------------------------------------------ sequences

    def open_sequence(self) -> int:
        slot = self.cache.open_sequence()
        self._forget_fed(slot)
        return slot

    def close_sequence(self, slot: int) -> None:
        self.cache.close_sequence(slot)
        self._forget_fed(slot)

    def _forget_fed(self, slot: int) -> None:
        """What the device holds as the next input of ``slot`` belongs to a sequence that is gone."""
        graphs = self.graphs
        if graphs is not None and graphs.fed is not None and slot in graphs.fed:
            graphs.fed = None

    def reserve(self, slot: int, tokens: int) -> None:
        """Set pages aside so that ``slot`` can grow to ``tokens`` tokens without asking again."""
        self.cache.reserve(slot, tokens)

    def prepare(self, max_position: int) -> None:
        """Grow what depends on the longest sequence; captured graphs that read moved tables go."""
        if self.model.prepare(max_position) and self.graphs is not None:
            self.graphs.drop()

    # ------------------------------------------------------------------ the step

    def make_context(self, entries) -> StepContext:
        cache = self.cache
        starts = [cache.lengths[e.slot] for e in entries]
        arrays = plan_step(entries, starts, self.model.spec.vocab_size)
        for e in entries:
            cache.reserve(e.slot, cache.lengths[e.slot] + len(e.tokens))
        for e in entries:
            cache.advance(e.slot, len(e.tokens))
        cache.sync_table()
        dev = upload(arrays, self.device)
        max_kv = int(arrays["seq_kv_len"].max())
        self.prepare(max_kv)
        return StepContext(
            n_tokens=int(arrays["tokens"].size), n_seqs=len(entries),
            tokens=dev["tokens"], tok_pos=dev["tok_pos"], tok_slot=dev["tok_slot"],
            seq_slot=dev["seq_slot"], seq_q_start=dev["seq_q_start"], seq_q_len=dev["seq_q_len"],
            seq_kv_len=dev["seq_kv_len"], want_rows=dev["want_rows"],
            tile_seq=dev["tile_seq"], tile_first=dev["tile_first"],
            block_seq=dev["block_seq"], block_first=dev["block_first"],
            max_q_len=int(arrays["seq_q_len"].max()), max_kv_len=max_kv,
            cache=cache, status=self.status, host=arrays)

    @torch.inference_mode()
    def step(self, entries) -> torch.Tensor:
        """Run one step; ``entries`` is a list of ``StepEntry``.  Returns ``[wanted, vocab]`` float32."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if self.graphs is not None:
            self.graphs.fed = None
        cache = self.cache
        before = [(e.slot, cache.lengths[e.slot]) for e in entries]
        try:
            ctx = self.make_context(entries)
            return self.model.forward(ctx, ctx.want_rows)
        except BaseException:
            # a step that raises leaves every sequence as long as it was: tokens whose keys were
            # never (or only partly) written are not counted, and later steps do not read them
            for slot, length in before:
                if cache.slots.is_held(slot):
                    cache.lengths[slot] = length
            raise

    @torch.inference_mode()
    def step_and_select(self, entries, sampler, temperatures, keys, positions) -> list:
        """One step plus token selection (the logits wanted are each entry's last place).

        Steps in which every sequence brings one token run as a captured graph that feeds itself;
        anything else runs the eager step and the sampler.  Both run the same kernels."""
        return self.start_step(entries, sampler, temperatures, keys, positions).result()

    @torch.inference_mode()
    def start_step(self, entries, sampler, temperatures, keys, positions) -> DrawnTokens:
        """``step_and_select`` without the wait: launches the step and returns a handle whose
        ``result()`` gives the drawn tokens.  An entry whose token is ``FED`` goes on from the token the
        device drew for it in the step before, which the host need not have seen yet; that is what
        lets a step be launched before its predecessor's tokens are read."""
        single = self.graphs is not None and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        if not single:
            if any(t is FED for e in entries for t in e.tokens):
                raise ValueError("only a captured single-token step can go on from device-held tokens")
            return DrawnTokens(ready=sampler.select(self.step(entries), temperatures, keys, positions))
        self.decode_tokens(entries, temperatures, keys)
        return self.graphs.fetch(len(entries))

    @torch.inference_mode()
    def decode_tokens(self, entries, temperatures, keys) -> torch.Tensor:
        """Graph path of ``step_and_select``; returns the drawn tokens on the device."""
        cache, graphs = self.cache, self.graphs
        slots = tuple(e.slot for e in entries)
        for e in entries:
            cache.reserve(e.slot, cache.lengths[e.slot] + 1)
        lengths = [cache.lengths[s] for s in slots]
        # the device may go on from what it drew itself only for the very same sequences at the
        # very lengths it left them at; anything else (another batch, a slot that was closed and
        # opened again, a step that came in between) is loaded from the host
        held = graphs.fed == slots and graphs.fed_lengths == lengths
        unknown = any(e.tokens[0] is FED for e in entries)
        if unknown and not held:
            raise RuntimeError("a step asked to go on from device-held tokens, but the device does not "
                               "hold the next inputs of exactly these sequences")
        if unknown and not self.self_feeding:
            graphs.load(slots, None, lengths, temperatures, keys)     # all but the tokens from the host
        elif not held or not self.self_feeding:
            for e in entries:
                if not 0 <= e.tokens[0] < self.model.spec.vocab_size:
                    raise ValueError(f"token id {e.tokens[0]} is outside the vocabulary")
            graphs.load(slots, [e.tokens[0] for e in entries], lengths, temperatures, keys)
        cache.sync_table()
        longest = max(lengths) + 1
        self.prepare(longest)
        out = graphs.replay(len(slots), longest)
        for s in slots:
            cache.advance(s, 1)
        graphs.fed_lengths = [n + 1 for n in lengths]
        return out

    def check_status(self) -> None:
        """Raise if a kernel flagged a bad input since the last check (reads one int from the device)."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            problems = []
            if code & 1:
                problems.append("a token id outside the vocabulary reached the embedding")
            if code & 2:
                problems.append("a row of logits held no finite value")
            if code & 4:
                problems.append("a wait inside the tensor-core product ran out of time")
            if code & 8:
                problems.append("a wait inside the decode attention kernel ran out of time")
            if code & 16:
                problems.append("a wait inside the tensor-core prefill attention kernel ran out of time")
            raise RuntimeError("; ".join(problems) or f"device status {code}")
