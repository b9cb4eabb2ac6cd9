"""One layer with the layer sizes of Qwen3-4B (hidden 2560, 32 query heads over 8 key/value heads of
128, intermediate 9728) and an odd vocabulary: the kernels' real tile, split and stage choices, which
the tiny configurations never reach, against the plain implementation."""

import pytest
import torch

import plain_qwen3 as plain
from gpu_helpers import DTYPES, assert_close
from tiny import random_prompt

pytestmark = pytest.mark.gpu

REAL = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=1, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=9728, vocab_size=4099, rope_theta=5e6, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=4096, hidden_act="silu",
)

_made = {}


def real_case(tmp_path_factory):
    if not _made:
        from starter_b200.config import config_from_dict
        from starter_b200.weights import write_model_folder

        folder = write_model_folder(str(tmp_path_factory.mktemp("real")), config_from_dict(REAL), 3,
                                    torch.bfloat16)
        cfg, w = plain.read_model_folder(folder)
        _made["case"] = (folder, cfg, w)
    return _made["case"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_real_layer_sizes_whole_stepwise_and_batched(tmp_path_factory, dtype):
    from starter_b200.engine import ModelRunner, StepEntry, load_model

    folder, cfg, w = real_case(tmp_path_factory)
    runner = ModelRunner(load_model(folder, dtype), max_tokens=64 * 40, max_sequences=16)
    vocab = cfg["vocab_size"]
    seqs = [random_prompt(n, vocab, 500 + n) for n in (300, 70, 9)]
    want = [plain.plain_forward(cfg, w, s) for s in seqs]
    # whole
    slot = runner.open_sequence()
    got = runner.step([StepEntry(slot, seqs[0], list(range(300)))])
    runner.close_sequence(slot)
    assert_close(got, want[0], dtype, "real sizes, 300 tokens whole")
    # a batch of unequal prompts, then nine single-token steps of all three (rows = 3: the few-row
    # kernels), the shortest leaving first
    slots = [runner.open_sequence() for _ in seqs]
    heads = [280, 61, 3]
    out = runner.step([StepEntry(s, q[:h], [h - 1]) for s, q, h in zip(slots, seqs, heads)])
    for i in range(3):
        assert_close(out[i:i + 1], want[i][heads[i] - 1][None], dtype, f"real sizes, batched prompt {i}")
    for step in range(9):
        live = [i for i in range(3) if heads[i] + step < len(seqs[i])]
        out = runner.step([StepEntry(slots[i], [seqs[i][heads[i] + step]], [0]) for i in live])
        for row, i in enumerate(live):
            assert_close(out[row:row + 1], want[i][heads[i] + step][None], dtype,
                         f"real sizes, request {i} step {step}")
    for s in slots:
        runner.close_sequence(s)
    runner.check_status()
    runner.cache.check()


def test_real_layer_sizes_graph_decode_of_a_full_batch(tmp_path_factory):
    """Sixteen sequences decoded through the captured, self-feeding step: the logits every replay
    leaves, against the plain implementation and against the eager step fed the same tokens."""
    from starter_b200 import Engine
    from starter_b200.engine import StepEntry
    from starter_b200.engine.generate import Request

    folder, cfg, w = real_case(tmp_path_factory)
    prompts = [random_prompt(5 + 7 * i, cfg["vocab_size"], 700 + i) for i in range(16)]
    engine = Engine(folder, dtype="bfloat16", max_batch=16)
    requests = [Request(list(p), 6) for p in prompts]
    loop = engine._ensure_room(requests, len(requests))
    loop.lookahead = False            # each step's logits are read before the next step runs
    graphs = engine.runner.graphs
    tokens, rows = [[] for _ in prompts], []
    for n, step_out in enumerate(loop.stream_batch(requests)):
        if n > 0:
            rows.append(graphs.logits[graphs.last_key].clone())
        for i in range(16):
            tokens[i].append(step_out[i])
    engine.runner.check_status()
    assert len(rows) == 5
    want = [plain.plain_forward(cfg, w, list(p) + t) for p, t in zip(prompts, tokens)]
    for step, got in enumerate(rows):
        ref = torch.stack([want[i][len(prompts[i]) + step] for i in range(16)])
        assert_close(got, ref, "bfloat16", f"captured step {step} of 16 sequences")
    # the eager step, fed the same tokens one by one, computes the same thing with the same kernels
    runner = engine.runner
    slots = [runner.open_sequence() for _ in prompts]
    runner.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
    for step, got in enumerate(rows):
        eager = runner.step([StepEntry(s, [t[step]], [0]) for s, t in zip(slots, tokens)])
        assert_close(eager, got, "bfloat16", f"eager against captured, step {step}")
    for s in slots:
        runner.close_sequence(s)


@pytest.mark.parametrize("n,grow", [(64, 5), (100, 3)])
def test_real_layer_sizes_many_unequal_sequences(tmp_path_factory, n, grow):
    """A batch of 64 (the widest of the usual tiles of every product, one part per sequence in the
    attention) and one of 100 (128-row tiles in the few-row product): the prompts in one step, then
    one eager and one captured single-token step, every row against the plain implementation."""
    from starter_b200.engine import ModelRunner, StepEntry, load_model

    folder, cfg, w = real_case(tmp_path_factory)
    vocab = cfg["vocab_size"]
    seqs = [random_prompt(3 + grow * i + 2, vocab, 1200 + i) for i in range(n)]     # prompt + 2 tokens
    want = [plain.plain_forward(cfg, w, s) for s in seqs]
    runner = ModelRunner(load_model(folder, "bfloat16"), max_tokens=n * 6 * 64, max_sequences=n)
    slots = [runner.open_sequence() for _ in seqs]
    heads = [len(s) - 2 for s in seqs]
    out = runner.step([StepEntry(s, q[:h], [h - 1]) for s, q, h in zip(slots, seqs, heads)])
    assert_close(out, torch.stack([want[i][heads[i] - 1] for i in range(n)]), "bfloat16", f"{n} prompts, last places")
    out = runner.step([StepEntry(s, [q[h]], [0]) for s, q, h in zip(slots, seqs, heads)])
    assert_close(out, torch.stack([want[i][heads[i]] for i in range(n)]), "bfloat16", f"{n} rows, eager step")
    runner.decode_tokens([StepEntry(s, [q[h + 1]], [0]) for s, q, h in zip(slots, seqs, heads)],
                         [0.0] * n, [0] * n)
    got = runner.graphs.logits[runner.graphs.last_key]
    assert got.shape[0] == n
    assert_close(got, torch.stack([want[i][heads[i] + 1] for i in range(n)]), "bfloat16", f"{n} rows, captured step")
    for s in slots:
        runner.close_sequence(s)
    runner.check_status()
    runner.cache.check()


def test_captured_decode_is_reproducible_over_many_steps(tmp_path_factory):
    """Two hundred self-feeding steps of eight unequal sequences, twice: the same tokens both times,
    no device status raised.  The sequences cross page edges and the length classes of the captured
    graphs on the way, and consecutive replays overlap at their seam, so anything a kernel reads
    before its dependent-launch wait that an earlier kernel still writes would show here."""
    from starter_b200 import Engine

    folder, cfg, w = real_case(tmp_path_factory)
    prompts = [random_prompt(3 + 17 * i, cfg["vocab_size"], 900 + i) for i in range(8)]
    engine = Engine(folder, dtype="bfloat16", max_batch=8)
    first = list(engine.generate(prompts, 200))
    engine.runner.check_status()
    again = list(engine.generate(prompts, 200))
    engine.runner.check_status()
    assert first == again
    assert len({tuple(step) for step in first}) > 20      # not stuck on one token


WIDE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=1, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
    intermediate_size=17408, vocab_size=1031, rope_theta=1e6, rms_norm_eps=1e-6,
    tie_word_embeddings=False, max_position_embeddings=4096, hidden_act="silu",
)


def test_a_layer_of_the_widest_model_size(tmp_path_factory):
    """Hidden 5120, 40 query heads over 8 key/value heads, intermediate 17408, an untied head (the
    14B row of the measurement table): other tile counts, split choices and cluster sizes than the 4B
    layer.  A prompt whole, then unequal sequences through the captured step, against the plain model."""
    from starter_b200 import Engine
    from starter_b200.config import config_from_dict
    from starter_b200.engine import ModelRunner, StepEntry, load_model
    from starter_b200.engine.generate import Request
    from starter_b200.weights import write_model_folder

    folder = write_model_folder(str(tmp_path_factory.mktemp("wide")), config_from_dict(WIDE), 5, torch.bfloat16)
    cfg, w = plain.read_model_folder(folder)
    vocab = cfg["vocab_size"]
    runner = ModelRunner(load_model(folder, "bfloat16"), max_tokens=64 * 8, max_sequences=4)
    seq = random_prompt(150, vocab, 21)
    slot = runner.open_sequence()
    got = runner.step([StepEntry(slot, seq, list(range(150)))])
    runner.close_sequence(slot)
    assert_close(got, plain.plain_forward(cfg, w, seq), "bfloat16", "widest layer, 150 tokens whole")
    runner.check_status()
    del runner
    prompts = [random_prompt(n, vocab, 30 + n) for n in (70, 9, 1)]
    engine = Engine(folder, dtype="bfloat16", max_batch=4)
    requests = [Request(list(p), 5) for p in prompts]
    loop = engine._ensure_room(requests, len(requests))
    loop.lookahead = False            # each step's logits are read before the next step runs
    graphs = engine.runner.graphs
    tokens, rows = [[] for _ in prompts], []
    for n, step_out in enumerate(loop.stream_batch(requests)):
        if n > 0:
            rows.append(graphs.logits[graphs.last_key].clone())
        for i in range(3):
            tokens[i].append(step_out[i])
    engine.runner.check_status()
    want = [plain.plain_forward(cfg, w, list(p) + t) for p, t in zip(prompts, tokens)]
    for step, got in enumerate(rows):
        ref = torch.stack([want[i][len(prompts[i]) + step] for i in range(3)])
        assert_close(got, ref, "bfloat16", f"widest layer, captured step {step}")
