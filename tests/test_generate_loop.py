"""The generation loop's decisions, with a runner and a sampler that need no device (no GPU)."""

import numpy as np
import pytest
import torch

from starter_b200.engine.generate import (Completion, GenerationLoop, Request, pages_held, plan_batches,
                                          tokens_held)
from starter_b200.sampling import SamplingParams, gumbel_noise, request_key

VOCAB = 50


class ScriptedRunner:
    """Keeps each sequence's tokens and answers with logits that make token ``f(sequence so far)`` win."""

    def __init__(self, slots=8):
        self.free = list(range(slots))[::-1]
        self.seqs = {}
        self.reserved = {}
        self.steps = []
        self.closed = []

    def open_sequence(self):
        slot = self.free.pop()
        self.seqs[slot] = []
        return slot

    def reserve(self, slot, tokens):
        self.reserved[slot] = tokens

    def close_sequence(self, slot):
        assert slot in self.seqs, "closed twice"
        del self.seqs[slot]
        self.closed.append(slot)
        self.free.append(slot)

    @staticmethod
    def next_token(seq):
        return (sum(seq) * 7 + len(seq)) % VOCAB

    def step(self, entries):
        self.steps.append([(e.slot, list(e.tokens), list(e.want)) for e in entries])
        rows = []
        for e in entries:
            for i, t in enumerate(e.tokens):
                self.seqs[e.slot].append(t)
                if i in e.want:
                    row = torch.zeros(VOCAB)
                    row[self.next_token(self.seqs[e.slot])] = 5.0
                    rows.append(row)
            assert len(self.seqs[e.slot]) <= self.reserved[e.slot]
        return torch.stack(rows)


class HostSampler:
    def select(self, logits, temperatures, keys, positions):
        out = []
        for row, t, key, pos in zip(logits.numpy(), temperatures, keys, positions):
            if t <= 0:
                out.append(int(np.argmax(row)))
            else:
                out.append(int(np.argmax(row / np.float32(t) + gumbel_noise(key, pos, row.size))))
        return out


def expected(prompt, n, stops=()):
    seq, out = list(prompt), []
    for _ in range(n):
        tok = ScriptedRunner.next_token(seq)
        out.append(tok)
        seq.append(tok)
        if tok in stops:
            break
    return out


def test_unequal_prompts_prefill_in_one_step_then_one_token_each():
    runner = ScriptedRunner()
    loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100)
    reqs = [Request([1, 2, 3, 4, 5], 4), Request([9, 8, 7], 4)]
    done = loop.run_batch(reqs)
    assert [d.tokens for d in done] == [expected(r.prompt, 4) for r in reqs]
    assert all(d.finish_reason == "length" for d in done)
    first = runner.steps[0]
    assert [len(t) for _, t, _ in first] == [5, 3] and [w for _, _, w in first] == [[4], [2]]
    assert all(len(t) == 1 and w == [0] for step in runner.steps[1:] for _, t, w in step)
    assert len(runner.steps) == 4            # the last drawn token is never fed back
    assert runner.seqs == {} and sorted(runner.closed) == [0, 1]


def test_a_sequence_that_stops_leaves_and_the_others_go_on():
    runner = ScriptedRunner()
    loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100)
    prompts = [[3, 1], [4, 4, 4], [2]]
    plain = [expected(p, 6) for p in prompts]
    stop = plain[1][2]                       # the second request stops at its third token
    reqs = [Request(p, 6, stop_token_ids={stop}) for p in prompts]
    done = loop.run_batch(reqs)
    for d, p in zip(done, prompts):
        want = expected(p, 6, {stop})
        assert d.tokens == want
        assert d.finish_reason == ("stop" if want[-1] == stop else "length")
    assert done[1].tokens == plain[1][:3]
    sizes = [len(step) for step in runner.steps]
    assert sizes[0] == 3 and sizes == sorted(sizes, reverse=True) and sizes[-1] < 3
    assert runner.seqs == {}


def test_max_new_tokens_one_and_zero():
    runner = ScriptedRunner()
    loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100)
    done = loop.run([Request([5, 6], 1), Request([7], 0), Request([1, 1, 1], 2)])
    assert done[0].tokens == expected([5, 6], 1) and done[1].tokens == [] and len(done[2].tokens) == 2
    assert len(runner.steps) == 2 and len(runner.steps[0]) == 2


def test_batches_follow_one_another_and_slots_are_used_again():
    runner = ScriptedRunner(slots=2)
    loop = GenerationLoop(runner, HostSampler(), max_batch=2, max_pages=100)
    prompts = [[i + 1] * (i + 1) for i in range(5)]
    done = loop.run([Request(p, 3) for p in prompts])
    assert [d.tokens for d in done] == [expected(p, 3) for p in prompts]
    assert len(runner.closed) == 5 and set(runner.closed) == {0, 1}


def test_plan_batches_respects_batch_size_pages_and_order():
    reqs = [Request([0] * 60, 5), Request([0] * 64, 2), Request([0] * 10, 0), Request([0] * 200, 1),
            Request([0] * 1, 1)]
    assert [tokens_held(r) for r in reqs] == [64, 65, 10, 200, 1]
    assert [pages_held(r) for r in reqs] == [1, 2, 1, 4, 1]
    assert plan_batches(reqs, max_batch=8, max_pages=100) == [[0, 1, 3, 4]]
    assert plan_batches(reqs, max_batch=2, max_pages=100) == [[0, 1], [3, 4]]
    assert plan_batches(reqs, max_batch=8, max_pages=4) == [[0, 1], [3], [4]]
    with pytest.raises(ValueError):
        plan_batches(reqs, max_batch=8, max_pages=3)


def test_a_draw_depends_on_seed_request_and_position_only():
    a = gumbel_noise(request_key(1, 0), 5, 64)
    assert np.array_equal(a, gumbel_noise(request_key(1, 0), 5, 64))
    for other in (gumbel_noise(request_key(2, 0), 5, 64), gumbel_noise(request_key(1, 1), 5, 64),
                  gumbel_noise(request_key(1, 0), 6, 64)):
        assert not np.array_equal(a, other)
    assert np.isfinite(a).all()

    def run(batch_prompts, numbers):
        runner = ScriptedRunner()
        loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100)
        reqs = [Request(p, 5, SamplingParams(temperature=3.0, seed=11), number=n)
                for p, n in zip(batch_prompts, numbers)]
        return [d.tokens for d in loop.run(reqs)]

    alone = run([[4, 2]], [7])
    together = run([[1], [4, 2], [3, 3, 3]], [0, 7, 2])
    assert together[1] == alone[0]


def test_temperature_draws_follow_the_softmax():
    logits = np.log(np.array([0.6, 0.3, 0.1], dtype=np.float32))
    counts = np.zeros(3)
    for pos in range(4000):
        counts[int(np.argmax(logits + gumbel_noise(request_key(5, 3), pos, 3)))] += 1
    assert np.abs(counts / 4000 - [0.6, 0.3, 0.1]).max() < 0.03


def test_slots_are_closed_when_a_step_fails():
    class Failing(ScriptedRunner):
        def step(self, entries):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().step(entries)

    runner = Failing()
    loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100)
    with pytest.raises(RuntimeError):
        loop.run_batch([Request([1, 2], 5), Request([3], 5)])
    assert runner.seqs == {}


# ----------------------------------------------------------------------------- one step of lookahead

class LookaheadRunner(ScriptedRunner):
    """A scripted runner that, like the device, keeps the token it drew as each sequence's next input
    and hands tokens out through handles; it writes down when steps are launched and when read."""

    def __init__(self, slots=8):
        super().__init__(slots)
        self.log = []
        self.drawn = {}          # slot -> the token drawn last for it (what the device would hold)
        self.count = 0

    def start_step(self, entries, sampler, temperatures, keys, positions):
        from starter_b200.engine.batch import FED, StepEntry

        single = all(len(e.tokens) == 1 for e in entries)
        number = self.count
        self.count += 1
        filled = []
        for e in entries:
            if e.tokens[0] is FED:
                assert single and e.slot in self.drawn, "no device-held token for this sequence"
                filled.append(StepEntry(e.slot, [self.drawn[e.slot]], e.want))
            else:
                filled.append(e)
        self.log.append(("launch", number, [e.tokens[0] is FED for e in entries]))
        tokens = sampler.select(self.step(filled), temperatures, keys, positions)
        for e, t in zip(entries, tokens):
            self.drawn[e.slot] = t
        runner = self

        class Handle:
            device_feeds = single

            def result(self):
                runner.log.append(("read", number))
                return tokens

        return Handle()


def test_the_next_step_is_launched_before_this_steps_tokens_are_read():
    runner = LookaheadRunner()
    loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100)
    prompts = [[3, 1, 4], [1, 5]]
    done = loop.run_batch([Request(p, 5) for p in prompts])
    assert [d.tokens for d in done] == [expected(p, 5) for p in prompts]
    # step 0 (the prompts) is read before step 1 goes out with host tokens; from then on every step
    # is launched, with device-held tokens, before the step before it is read; the last token needs
    # no step of its own (5 tokens: the prompt step and four more)
    assert runner.log == [
        ("launch", 0, [False, False]), ("read", 0),
        ("launch", 1, [False, False]),
        ("launch", 2, [True, True]), ("read", 1),
        ("launch", 3, [True, True]), ("read", 2),
        ("launch", 4, [True, True]), ("read", 3),
        ("read", 4),
    ]
    assert sorted(runner.closed) == [0, 1] and not runner.seqs


def test_no_lookahead_where_a_token_can_end_a_sequence_or_the_batch_changes():
    runner = LookaheadRunner()
    loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100)
    prompts = [[3, 1, 4], [1, 5]]
    # a stop token may end a sequence at any step: every step is read before the next goes out
    want = expected(prompts[0], 6)
    done = loop.run_batch([Request(prompts[0], 6, stop_token_ids={want[3]}), Request(prompts[1], 6)])
    assert done[0].tokens == want[:4] and done[0].finish_reason == "stop"
    assert done[1].tokens == expected(prompts[1], 6)
    launches = [e for e in runner.log if e[0] == "launch"]
    reads = [e for e in runner.log if e[0] == "read"]
    assert all(runner.log.index(("read", n)) < runner.log.index(launches[n + 1]) for n in range(4))
    # ... until the request that could stop has left; the other then runs ahead
    assert any(flags == [True] for _, _, flags in launches)
    # unequal lengths without stop tokens: the step in which one sequence ends is read before the
    # next (smaller) batch is launched with host tokens, and nothing runs for a finished sequence
    runner = LookaheadRunner()
    loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100)
    done = loop.run_batch([Request(prompts[0], 2), Request(prompts[1], 5)])
    assert [d.tokens for d in done] == [expected(prompts[0], 2), expected(prompts[1], 5)]
    assert runner.log == [
        ("launch", 0, [False, False]), ("read", 0),
        ("launch", 1, [False, False]), ("read", 1),       # request 0 ends here: no lookahead
        ("launch", 2, [False]),
        ("launch", 3, [True]), ("read", 2),
        ("launch", 4, [True]), ("read", 3),
        ("read", 4),
    ]
    # with the option off, every step is read before the next is launched, and the tokens are the same
    runner = LookaheadRunner()
    loop = GenerationLoop(runner, HostSampler(), max_batch=4, max_pages=100, lookahead=False)
    done = loop.run_batch([Request(p, 5) for p in prompts])
    assert [d.tokens for d in done] == [expected(p, 5) for p in prompts]
    assert [e[0] for e in runner.log] == ["launch", "read"] * 5
