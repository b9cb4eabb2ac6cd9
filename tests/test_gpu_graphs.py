"""The captured, self-feeding one-token step (the path generation takes) against the plain
implementation: long runs that cross page edges and the length classes of the captured graphs, the
logits each replay leaves, slots that are used again by one-token prompts."""

import pytest
import torch

import plain_qwen3 as plain
from gpu_helpers import DTYPES, assert_close, model_case
from tiny import random_prompt

pytestmark = pytest.mark.gpu


def run_and_record(engine, prompts, new_tokens):
    """Greedy generation through the loop that serves ``Engine.complete``; returns the tokens of each
    request and, for every captured step, the logits the graph left for each live request."""
    from starter_b200.engine.generate import GenerationLoop, Request

    requests = [Request(list(p), new_tokens) for p in prompts]
    loop = engine._ensure_room(requests, len(requests))
    loop.lookahead = False            # each step's logits are read before the next step runs
    assert isinstance(loop, GenerationLoop)
    graphs = engine.runner.graphs
    tokens = [[] for _ in prompts]
    rows = [[] for _ in prompts]       # rows[i][t]: logits that chose token t + 1 of request i
    keys_used = set()
    for n, step_out in enumerate(loop.stream_batch(requests)):
        live = sorted(step_out)
        if n > 0:
            keys_used.add(graphs.last_key)
            logits = graphs.logits[graphs.last_key]
            for row, i in enumerate(live):
                rows[i].append(logits[row].clone())
        for i in live:
            tokens[i].append(step_out[i])
    return tokens, rows, keys_used


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_captured_runs_against_the_plain_implementation(tmp_path_factory, name, dtype):
    from starter_b200 import Engine

    folder, cfg, w = model_case(tmp_path_factory, name)
    vocab = cfg["vocab_size"]
    lengths, new = (3, 60, 120), 170
    prompts = [random_prompt(n, vocab, 400 + n) for n in lengths]
    engine = Engine(folder, dtype=dtype, max_batch=4)
    tokens, rows, keys_used = run_and_record(engine, prompts, new)
    engine.runner.check_status()
    # every request crossed the page edges at 64, 128 (and 192, 256) tokens, and the batch went
    # through at least three length classes, each a graph of its own
    assert len({pages for _, pages in keys_used}) >= 3
    for i, prompt in enumerate(prompts):
        assert len(tokens[i]) == new and len(rows[i]) == new - 1
        seq = list(prompt) + tokens[i]
        want = plain.plain_forward(cfg, w, seq)
        # the replay that drew token t + 1 ran token t, which sits at place len(prompt) + t
        at = len(prompt)
        assert_close(torch.stack(rows[i]), want[at:at + new - 1], dtype,
                     f"{name} captured step, request {i} (prompt of {len(prompt)})")
        if dtype == "float32":
            assert tokens[i] == plain.plain_generate(cfg, w, prompt, new), f"request {i}"
    # the same through the reference-style entry point (which launches a step ahead of reading)
    again = list(engine.generate(prompts, new))
    assert [[s[i] for s in again] for i in range(len(prompts))] == tokens


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_token_prompts_in_a_slot_that_was_just_used(tmp_path_factory, dtype):
    """A prompt of one token runs as a captured step from its first token on.  The slot it gets was
    held a moment ago by another sequence whose next input the device still holds: none of that
    (token, position, length, sampling settings) may reach the new sequence."""
    from starter_b200 import Engine

    folder, cfg, w = model_case(tmp_path_factory, "A")
    vocab = cfg["vocab_size"]
    engine = Engine(folder, dtype=dtype, max_batch=4)
    margin = 2e-5 if dtype == "float32" else 3e-2

    def check(prompt_sets, new):
        for prompts in prompt_sets:
            steps = list(engine.generate(prompts, new))
            graphs, cache = engine.runner.graphs, engine.runner.cache
            for i, prompt in enumerate(prompts):
                mine = [s[i] for s in steps]
                if dtype == "float32":
                    assert mine == plain.plain_generate(cfg, w, prompt, new), (prompts, i)
                seq = list(prompt)
                for tok in mine:
                    logits = plain.plain_forward(cfg, w, seq)[-1]
                    assert logits[tok].item() >= logits.max().item() - margin * max(1.0, logits.abs().max().item())
                    seq.append(tok)
            assert cache.slots.held_count == 0

    one, other = [[5]], [[200]]
    longer = [random_prompt(9, vocab, 1)]
    # the same one-token prompt twice; another one after it; one after a longer prompt; two at once
    # after one; and a one-token prompt next to a longer one in one batch
    check([one, one, other, longer, one, [[7], [9]], other, [[11], random_prompt(6, vocab, 2)], one], 5)

    # the device-held length of a fed slot always is the cache's own
    from starter_b200.engine import StepEntry
    runner = engine.runner
    slot = runner.open_sequence()
    runner.reserve(slot, 40)
    tok = 3
    for step in range(6):
        out = runner.decode_tokens([StepEntry(slot, [tok], [0])], [0.0], [0])
        tok = int(out.tolist()[0])
        held = int(runner.graphs._field("kv_len", 1).tolist()[0])
        assert held == runner.cache.lengths[slot] + 1 == step + 2
    runner.close_sequence(slot)
    slot2 = runner.open_sequence()
    assert slot2 == slot                                  # the slot comes straight back
    runner.decode_tokens([StepEntry(slot2, [3], [0])], [0.0], [0])
    assert int(runner.graphs._field("kv_len", 1).tolist()[0]) == 2
    runner.close_sequence(slot2)
    runner.check_status()


def test_a_step_that_raises_leaves_the_lengths_as_they_were(tmp_path_factory):
    from starter_b200.engine import StepEntry

    folder, cfg, w = model_case(tmp_path_factory, "A")
    from starter_b200.engine import ModelRunner, load_model
    runner = ModelRunner(load_model(folder, "float32"), max_tokens=64 * 4, max_sequences=2)
    a, b = runner.open_sequence(), runner.open_sequence()
    prompt = random_prompt(10, cfg["vocab_size"], 1)
    runner.step([StepEntry(a, prompt[:6], [])])
    with pytest.raises(Exception):
        # the second sequence asks for more pages than the cache has: nothing of the step counts
        runner.step([StepEntry(a, prompt[6:8], [0]), StepEntry(b, [1] * (64 * 4), [0])])
    assert runner.cache.lengths[a] == 6 and runner.cache.lengths[b] == 0
    got = runner.step([StepEntry(a, prompt[6:], [0, 1, 2, 3])])
    assert_close(got, plain.plain_forward(cfg, w, prompt)[6:], "float32", "after a refused step")
    runner.close_sequence(a)
    runner.close_sequence(b)
    runner.cache.check()
