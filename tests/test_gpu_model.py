"""The engine against the plain implementation, on the GPU, in float32 and in bfloat16: every way of
cutting the same requests into steps and batches must give the same logits."""

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from gpu_helpers import DTYPES, assert_close, model_case, runner_for, tolerance
from tiny import random_prompt

pytestmark = pytest.mark.gpu

CONFIGS = ["A", "B", "C"]


def all_places(n):
    return list(range(n))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_each_request_alone_and_whole(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    for length, seed in ((1, 1), (7, 2), (64, 3), (65, 4), (150, 5)):
        prompt = random_prompt(length, cfg["vocab_size"], seed)
        slot = runner.open_sequence()
        got = runner.step([StepEntry(slot, prompt, all_places(length))])
        runner.close_sequence(slot)
        assert_close(got, plain.plain_forward(cfg, w, prompt), dtype, f"{name} whole, length {length}")
    runner.check_status()
    runner.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_last_32_tokens_one_by_one(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    for length in (33, 90):
        prompt = random_prompt(length, cfg["vocab_size"], 10 + length)
        want = plain.plain_forward(cfg, w, prompt)
        slot = runner.open_sequence()
        head = length - 32
        rows = [runner.step([StepEntry(slot, prompt[:head], all_places(head))])]
        for t in prompt[head:]:
            rows.append(runner.step([StepEntry(slot, [t], [0])]))
        runner.close_sequence(slot)
        got = torch.cat(rows)
        assert_close(got, want, dtype, f"{name} last 32 one by one, length {length}")
        # what is special about a place shows in the first wrong row: name it
        assert_close(got[head:head + 1], want[head:head + 1], dtype, "the first single-token step")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_unequal_batches_one_after_another(tmp_path_factory, name, dtype):
    """Batches of unequal prompts whose shorter requests end earlier; the second batch uses the slots
    and pages the first gave back; a chunk of several tokens goes into a cache that already holds some."""
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    vocab = cfg["vocab_size"]
    batches = [
        # (prompt length, tokens decoded one by one afterwards)
        [(70, 9), (5, 3), (33, 12), (1, 6)],
        [(2, 40), (129, 2), (64, 5)],
        [(17, 0), (63, 3)],
    ]
    seed = 100
    for batch in batches:
        seqs, slots, got = [], [], []
        for plen, extra in batch:
            seed += 1
            seqs.append(random_prompt(plen + extra, vocab, seed))
            slots.append(runner.open_sequence())
            got.append([])
        first = runner.step([StepEntry(slots[i], seqs[i][:plen], all_places(plen))
                             for i, (plen, _) in enumerate(batch)])
        offset = 0
        for i, (plen, _) in enumerate(batch):
            got[i].append(first[offset:offset + plen])
            offset += plen
        live = [i for i, (_, extra) in enumerate(batch) if extra > 0]
        for i, (_, extra) in enumerate(batch):
            if extra == 0:
                runner.close_sequence(slots[i])
        step = 0
        while live:
            out = runner.step([StepEntry(slots[i], [seqs[i][batch[i][0] + step]], [0]) for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1])
            step += 1
            for i in [i for i in live if batch[i][1] == step]:
                runner.close_sequence(slots[i])
            live = [i for i in live if batch[i][1] > step]
        for i, seq in enumerate(seqs):
            assert_close(torch.cat(got[i]), plain.plain_forward(cfg, w, seq), dtype,
                         f"{name} batch {batch}, request {i}")
        runner.cache.check()
    assert runner.cache.slots.held_count == 0 and runner.cache.pages.held_count == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_chunks_into_a_cache_that_already_holds_tokens(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    prompt = random_prompt(140, cfg["vocab_size"], 77)
    want = plain.plain_forward(cfg, w, prompt)
    slot = runner.open_sequence()
    rows, at = [], 0
    for size in (3, 61, 1, 64, 11):
        rows.append(runner.step([StepEntry(slot, prompt[at:at + size], all_places(size))]))
        at += size
    runner.close_sequence(slot)
    assert_close(torch.cat(rows), want, dtype, f"{name} chunks 3+61+1+64+11")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_long_decoding_and_the_first_tokens(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    seq = random_prompt(200, cfg["vocab_size"], 31)
    want = plain.plain_forward(cfg, w, seq)
    slot = runner.open_sequence()
    rows = [runner.step([StepEntry(slot, [t], [0])]) for t in seq]
    runner.close_sequence(slot)
    got = torch.cat(rows)
    assert_close(got[:2], want[:2], dtype, f"{name} the first two tokens of a sequence")
    assert_close(got, want, dtype, f"{name} 200 single-token steps")


@pytest.mark.parametrize("dtype", DTYPES)
def test_only_wanted_places_come_back_in_order(tmp_path_factory, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, "B")
    runner = runner_for(tmp_path_factory, "B", dtype)
    a, b, c = (random_prompt(n, cfg["vocab_size"], 50 + n) for n in (9, 4, 6))
    slots = [runner.open_sequence() for _ in range(3)]
    got = runner.step([StepEntry(slots[0], a, [8, 2]), StepEntry(slots[1], b, []), StepEntry(slots[2], c, [5])])
    for s in slots:
        runner.close_sequence(s)
    wa, wc = plain.plain_forward(cfg, w, a), plain.plain_forward(cfg, w, c)
    assert_close(got, torch.stack([wa[8], wa[2], wc[5]]), dtype, "wanted places")
    s = runner.open_sequence()
    assert runner.step([StepEntry(s, a, [])]).shape == (0, cfg["vocab_size"])
    runner.close_sequence(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_scattered_and_reused_pages(tmp_path_factory, dtype):
    """A sequence whose pages are neither adjacent nor fresh: pages freed by others, full of their keys."""
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, "A")
    runner = runner_for(tmp_path_factory, "A", dtype)
    vocab = cfg["vocab_size"]
    fill = [runner.open_sequence() for _ in range(5)]
    for i, s in enumerate(fill):
        runner.step([StepEntry(s, random_prompt(64 * (1 + i % 2), vocab, i), [])])
    for s in (fill[1], fill[3]):
        runner.close_sequence(s)
    seq = random_prompt(250, vocab, 99)
    slot = runner.open_sequence()
    got = runner.step([StepEntry(slot, seq, all_places(len(seq)))])
    pages = runner.cache.owned_pages(slot)
    assert pages != sorted(pages) or pages != list(range(pages[0], pages[0] + len(pages)))
    assert_close(got, plain.plain_forward(cfg, w, seq), dtype, "scattered pages")
    for s in (fill[0], fill[2], fill[4], slot):
        runner.close_sequence(s)
    runner.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, name, dtype):
    from starter_b200 import Engine

    folder, cfg, w = model_case(tmp_path_factory, name)
    lengths = [5, 3] if name == "A" else [7, 4, 1]
    new = 4 if name == "A" else 6
    prompts = [random_prompt(n, cfg["vocab_size"], 200 + n) for n in lengths]
    engine = Engine(folder, dtype=dtype)
    steps = list(engine.generate(prompts, new))
    assert len(steps) == new and all(len(s) == len(prompts) for s in steps)
    again = list(engine.generate(prompts, new))          # nothing carries over between calls
    assert again == steps
    margin = tolerance(dtype, torch.ones(1)) * 2
    for i, prompt in enumerate(prompts):
        mine = [s[i] for s in steps]
        seq = list(prompt)
        for tok in mine:
            logits = plain.plain_forward(cfg, w, seq)[-1]
            # the reference's own rule for a right token: within a margin of the oracle's maximum
            # on the engine's own prefix (QWEN_ENGINE_CONTRACT.md:105-123); the margin here is the
            # logit tolerance, not 2.0
            assert logits[tok].item() >= logits.max().item() - margin
            seq.append(tok)
    if dtype == "float32":
        want = [plain.plain_generate(cfg, w, p, new) for p in prompts]
        assert [[s[i] for s in steps] for i in range(len(prompts))] == want


def test_temperature_stop_tokens_and_batches_through_the_entry_point(tmp_path_factory):
    from starter_b200 import Engine

    folder, cfg, w = model_case(tmp_path_factory, "B")
    prompts = [random_prompt(n, cfg["vocab_size"], 300 + n) for n in (7, 4, 1, 12, 3)]
    engine = Engine(folder, dtype="float32", max_batch=3)
    done = engine.complete(prompts, 6, temperature=0.8, seed=42)
    want = [plain.plain_generate(cfg, w, p, 6, 0.8, 42, i) for i, p in enumerate(prompts)]
    assert [d.tokens for d in done] == want
    assert len({tuple(t) for t in want}) > 1
    stop = want[1][2]
    done = engine.complete(prompts, 6, temperature=0.8, seed=42, stop_token_ids=[stop])
    for i, d in enumerate(done):
        ref = plain.plain_generate(cfg, w, prompts[i], 6, 0.8, 42, i, stop_tokens=(stop,))
        assert d.tokens == ref and d.finish_reason == ("stop" if ref[-1] == stop else "length")
    assert done[1].tokens == want[1][:3]
    assert engine.runner.cache.slots.held_count == 0
    engine.runner.cache.check()


@pytest.mark.parametrize("name", CONFIGS)
def test_bfloat16_engine_against_the_plain_implementation_run_in_bfloat16(tmp_path_factory, name):
    """The plain implementation with bfloat16 weights and activations rounds where the reference
    rounds (it is held to the reference's own bfloat16 run in tests/test_plain.py); the bfloat16
    engine is held to it, whole and one token at a time, as to the float32 oracle."""
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, name)
    w16 = {k: v.to(torch.bfloat16) for k, v in w.items()}
    runner = runner_for(tmp_path_factory, name, "bfloat16")
    seq = random_prompt(150, cfg["vocab_size"], 61)
    want = plain.plain_forward(cfg, w16, seq)
    slot = runner.open_sequence()
    got = runner.step([StepEntry(slot, seq, all_places(len(seq)))])
    runner.close_sequence(slot)
    assert_close(got, want, "bfloat16", f"{name} whole, against the plain bfloat16 run")
    slot = runner.open_sequence()
    rows = [runner.step([StepEntry(slot, seq[:100], all_places(100))])]
    rows += [runner.step([StepEntry(slot, [t], [0])]) for t in seq[100:]]
    runner.close_sequence(slot)
    assert_close(torch.cat(rows), want, "bfloat16", f"{name} 100 + 50 x 1, against the plain bfloat16 run")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_prompts_long_enough_for_the_prompt_product(tmp_path_factory, name, dtype):
    """Steps of 512 rows and more take other kernels in bfloat16 (the CTA-pair product with its gated
    and residual epilogues, 256-query attention blocks): one long prompt whole, two long prompts of
    unequal length packed into one step, and a long prompt followed by a short chunk and single
    tokens, all against the plain implementation."""
    from starter_b200 import ops
    from starter_b200.engine import StepEntry

    _, cfg, w = model_case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype, max_tokens=64 * 48)
    a = random_prompt(700, cfg["vocab_size"], 71)
    b = random_prompt(ops.PROMPT_MIN_ROWS + 1, cfg["vocab_size"], 72)
    want_a, want_b = plain.plain_forward(cfg, w, a), plain.plain_forward(cfg, w, b)
    slot = runner.open_sequence()
    got = runner.step([StepEntry(slot, a, all_places(len(a)))])
    runner.close_sequence(slot)
    assert_close(got, want_a, dtype, f"{name} one prompt of {len(a)}")
    sa, sb = runner.open_sequence(), runner.open_sequence()
    got = runner.step([StepEntry(sa, a, [0, 350, 699]), StepEntry(sb, b, all_places(len(b)))])
    runner.close_sequence(sa)
    runner.close_sequence(sb)
    assert_close(got[:3], want_a[[0, 350, 699]], dtype, f"{name} the longer of two packed prompts")
    assert_close(got[3:], want_b, dtype, f"{name} the shorter of two packed prompts")
    slot = runner.open_sequence()
    rows = [runner.step([StepEntry(slot, a[:600], all_places(600))]),
            runner.step([StepEntry(slot, a[600:690], all_places(90))])]
    rows += [runner.step([StepEntry(slot, [t], [0])]) for t in a[690:]]
    runner.close_sequence(slot)
    assert_close(torch.cat(rows), want_a, dtype, f"{name} 600 + 90 + 10 x 1")
    runner.check_status()
    runner.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_long_sequence_decodes_through_many_parts(tmp_path_factory, dtype):
    """One sequence of 6,000 tokens: alone it cannot fill the GPU from a cluster's 8 parts, so its
    one-token steps cut the keys into many parts that meet in scratch memory and a merge kernel
    (the choice is asserted, so that the test keeps covering that path); the prompt before them walks
    94 pages through the prompt attention and several groups of row tiles through the prompt product."""
    from starter_b200 import ops
    from starter_b200.engine import StepEntry

    name = "A"
    _, cfg, w = model_case(tmp_path_factory, name)
    groups = cfg["num_attention_heads"] // cfg["num_key_value_heads"]
    assert ops.decode_splits(1, cfg["num_key_value_heads"], groups, 16, kv_hint=5995) > ops.DECODE_CLUSTER_SPLITS
    runner = runner_for(tmp_path_factory, name, dtype, max_tokens=64 * 95)
    seq = random_prompt(6000, cfg["vocab_size"], 81)
    want = plain.plain_forward(cfg, w, seq)
    head = 5990
    slot = runner.open_sequence()
    rows = [runner.step([StepEntry(slot, seq[:head], [0, 1000, head - 1])])]
    rows += [runner.step([StepEntry(slot, [t], [0])]) for t in seq[head:]]
    runner.close_sequence(slot)
    got = torch.cat(rows)
    places = [0, 1000, head - 1] + list(range(head, len(seq)))
    assert_close(got, want[places], dtype, f"{name} 5,990 tokens and 10 x 1")
    runner.check_status()
    runner.cache.check()


@pytest.mark.parametrize("name", ["B", "C"])
def test_random_batches_of_short_and_long_prompts_generate_right_tokens(tmp_path_factory, name):
    """Generation in bfloat16 over batches drawn at random: 1 to 8 sequences, prompts of 1 to 700
    tokens in one batch (so prompt steps of every kernel class), 1 to 17 new tokens, batch after
    batch on one engine.  Every token drawn must be, by the plain float32 model on the engine's own
    prefix, within the logit tolerance of the best token."""
    import random

    from gpu_helpers import BF16_TOL
    from starter_b200 import Engine

    folder, cfg, w = model_case(tmp_path_factory, name)
    engine = Engine(folder, dtype="bfloat16", max_batch=8)
    rng = random.Random(11)
    for _ in range(5):
        n = rng.choice([1, 2, 3, 5, 8])
        prompts = [random_prompt(rng.choice([1, 2, 63, 65, 130, 300, 520, 700]), cfg["vocab_size"], rng.randrange(10 ** 6))
                   for _ in range(n)]
        new = rng.choice([1, 2, 5, 17])
        for prompt, done in zip(prompts, engine.complete(prompts, new)):
            seq = list(prompt)
            for tok in done.tokens:
                logits = plain.plain_forward(cfg, w, seq)[-1]
                margin = 2 * BF16_TOL * float(logits.abs().max())
                assert logits[tok].item() >= logits.max().item() - margin, (len(prompt), len(seq))
                seq.append(tok)
        assert engine.runner.cache.slots.held_count == 0
        engine.runner.cache.check()
        engine.runner.check_status()
