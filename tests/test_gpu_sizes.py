"""Odd sizes through the whole engine: head sizes in steps of 16 (and one that is only even), one to
seven query heads per key/value head, widths and vocabularies that are no power of two, with and
without head norms, tied and untied heads, a window.  Each against the plain implementation, in
float32 and bfloat16: a prompt whole, single-token steps, and generation through the captured step."""

import pytest
import torch

import plain_qwen3 as plain
from gpu_helpers import DTYPES, assert_close
from tiny import random_prompt

pytestmark = pytest.mark.gpu


def cfg(layers, hidden, heads, kv_heads, head_dim, inter, vocab, theta=1e5, eps=1e-6, tied=True, **more):
    out = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=layers,
               hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
               intermediate_size=inter, vocab_size=vocab, rope_theta=theta, rms_norm_eps=eps,
               tie_word_embeddings=tied, max_position_embeddings=2048, hidden_act="silu")
    out.update(more)
    return out


SIZES = {
    "head80_groups7": cfg(2, 200, 7, 1, 80, 264, 509),
    "head112_groups3_untied": cfg(1, 136, 6, 2, 112, 320, 1021, theta=5e6, eps=1e-5, tied=False),
    "head192_one_head": cfg(2, 72, 1, 1, 192, 100, 251, theta=1e4),
    "head256_groups2_window": cfg(3, 96, 4, 2, 256, 192, 777, use_sliding_window=True, sliding_window=40,
                                  max_window_layers=1),
    "head24_only_even": cfg(2, 120, 5, 5, 24, 136, 333),
    "head64_no_head_norm": cfg(2, 328, 10, 2, 64, 704, 4099, qk_norm=False),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SIZES))
def test_odd_sizes_whole_stepwise_and_generated(tmp_path_factory, name, dtype):
    from starter_b200 import Engine
    from starter_b200.config import config_from_dict
    from starter_b200.engine import StepEntry
    from starter_b200.engine.generate import Request
    from starter_b200.weights import write_model_folder

    folder = write_model_folder(str(tmp_path_factory.mktemp(name)), config_from_dict(SIZES[name]), 11,
                                torch.float32)
    c, w = plain.read_model_folder(folder)
    vocab = c["vocab_size"]
    engine = Engine(folder, dtype=dtype, max_batch=4, max_tokens=64 * 16)
    runner = engine.runner
    seq = random_prompt(90, vocab, 5)
    want = plain.plain_forward(c, w, seq)
    slot = runner.open_sequence()
    got = runner.step([StepEntry(slot, seq[:70], list(range(70)))])
    rows = [got] + [runner.step([StepEntry(slot, [t], [0])]) for t in seq[70:]]
    runner.close_sequence(slot)
    assert_close(torch.cat(rows), want, dtype, f"{name}: 70 tokens whole, then 20 one by one")
    # generation: unequal prompts through the captured step, every replay's logits
    prompts = [random_prompt(n, vocab, 40 + n) for n in (66, 5, 1)]
    requests = [Request(list(p), 7) for p in prompts]
    loop = engine._ensure_room(requests, len(requests))
    loop.lookahead = False            # each step's logits are read before the next step runs
    graphs = runner.graphs
    tokens, logits = [[] for _ in prompts], []
    for n, step_out in enumerate(loop.stream_batch(requests)):
        if n > 0:
            logits.append(graphs.logits[graphs.last_key].clone())
        for i in range(3):
            tokens[i].append(step_out[i])
    runner.check_status()
    full = [plain.plain_forward(c, w, list(p) + t) for p, t in zip(prompts, tokens)]
    for step, got in enumerate(logits):
        ref = torch.stack([full[i][len(prompts[i]) + step] for i in range(3)])
        assert_close(got, ref, dtype, f"{name}: captured step {step}")
    if dtype == "float32":
        assert tokens == [plain.plain_generate(c, w, p, 7) for p in prompts]
    runner.cache.check()
