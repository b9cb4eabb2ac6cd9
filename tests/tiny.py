"""The tiny configurations the tests run: they differ in every size and option."""

import os

import torch

TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=4096, hidden_act="silu",
    use_sliding_window=False, sliding_window=None,
)

TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
    intermediate_size=160, vocab_size=300, rope_theta=1e6, rms_norm_eps=1e-5,
    tie_word_embeddings=False, max_position_embeddings=2048, hidden_act="silu",
    use_sliding_window=False, sliding_window=None,
)

# head_dim 48 (a step of 16 that is no power of two), one key/value head per query head, an odd
# vocabulary, and a window of 8 keys on the last two of four layers
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=4, hidden_size=80, num_attention_heads=5, num_key_value_heads=5, head_dim=48,
    intermediate_size=176, vocab_size=515, rope_theta=5e6, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=1024, hidden_act="silu",
    use_sliding_window=True, sliding_window=8, max_window_layers=2,
)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def make_folder(tmp_path, name, seed=0, dtype=torch.float32, **overrides):
    """Write a random-weights model folder for a tiny configuration and return its path."""
    from starter_b200.config import config_from_dict
    from starter_b200.weights import write_model_folder

    raw = dict(TINY[name])
    raw.update(overrides)
    path = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    return write_model_folder(path, config_from_dict(raw), seed, dtype)


def random_prompt(length, vocab, seed):
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=gen).tolist()
