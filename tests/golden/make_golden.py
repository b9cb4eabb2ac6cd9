"""Runs the reference's OWN forward code (engine/engine.py of alvinyuwen/starter) on the CPU in
float32 and in bfloat16 on tiny random models and stores its logits, so that tests can hold the plain
implementation (tests/plain_qwen3.py) against them without the reference being present.

    python tests/golden/make_golden.py /path/to/reference

The reference's ``Engine.__init__`` loads weights through a model library whose installed version
no longer has ``config.rope_theta`` (engine/engine.py:146), so the engine object is made with
``Engine.__new__`` and the attributes ``__init__`` would set (engine/engine.py:139-235) are filled
from a model folder written by ``starter_b200.weights.write_model_folder``.  Only the reference's
own functions compute: ``_grow_rope``, ``_ensure_shape``, ``_forward_prefill`` (hence ``_block``,
``rms_norm``, ``apply_rope``, ``_sdpa``).  It returns logits of the last position only, so every
position is obtained by running every prefix.  Output: ``reference_logits.json`` with, per case,
the config, the seed, the prompt, the float32 logits ``[T, vocab]`` rounded to 9 significant digits
and ``logits_bf16``: the same run with the reference's ``LOAD_DTYPE`` left at bfloat16
(engine/engine.py:41-43), which pins where the reference rounds to its working type.
"""

import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tiny import TINY, make_folder, random_prompt  # noqa: E402
import plain_qwen3 as plain  # noqa: E402

CASES = [("A", 11, 9), ("B", 12, 7), ("C", 13, 6)]  # (config, weight seed, prompt length)


def reference_engine(ref_root, cfg, w, dtype=torch.float32):
    if os.path.join(ref_root, "engine") not in sys.path:
        sys.path.insert(0, os.path.join(ref_root, "engine"))
    import engine as ref  # the reference's engine/engine.py

    ref.DEVICE = "cpu"
    ref.LOAD_DTYPE = dtype
    w = {k: v.to(dtype) for k, v in w.items()}
    e = ref.Engine.__new__(ref.Engine)
    e.LAYERS = cfg["num_hidden_layers"]
    e.HIDDEN = cfg["hidden_size"]
    e.HEADS = cfg["num_attention_heads"]
    e.KV_HEADS = cfg["num_key_value_heads"]
    e.HEAD_DIM = cfg["head_dim"]
    e.GROUPS = e.HEADS // e.KV_HEADS
    e.EPS = cfg["rms_norm_eps"]
    e.THETA = cfg["rope_theta"]
    e.SCALE = e.HEAD_DIM ** -0.5
    e.embed = w["model.embed_tokens.weight"]
    e.final_norm_w = w["model.norm.weight"]
    e.lm_head_w = e.embed if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    e.layers = []
    for i in range(e.LAYERS):
        p = f"model.layers.{i}."
        e.layers.append({
            "idx": i,
            "in_ln": w[p + "input_layernorm.weight"],
            "qkv": torch.cat([w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                              w[p + "self_attn.v_proj.weight"]], dim=0).contiguous(),
            "q_norm": w[p + "self_attn.q_norm.weight"],
            "k_norm": w[p + "self_attn.k_norm.weight"],
            "o": w[p + "self_attn.o_proj.weight"],
            "post_ln": w[p + "post_attention_layernorm.weight"],
            "gate_up": torch.cat([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]], dim=0).contiguous(),
            "down": w[p + "mlp.down_proj.weight"],
        })
    e.transposed = {}
    e.dtype = dtype
    e.cuda = False
    e.q_size = e.HEADS * e.HEAD_DIM
    e.kv_size = e.KV_HEADS * e.HEAD_DIM
    e.rope_len = 0
    e.cos_table = e.sin_table = None
    e._grow_rope(4096)
    e.cache_k = e.cache_v = None
    e.capacity = e.batch = 0
    e.graph = e.g_token = e.g_pos = e.g_out = e.g_arange = None
    e.gqa = True
    e.time_probe = 0
    e.fused_norm = e.fused_rope = e.fused_swiglu = e.fused_attn = False
    e.fused_add_norm = e.fused_kv_cache = e.fused_norm_rope = False
    e.gemm_blocks = None
    e.gemm_choice = {}
    e.prefill_fused = True
    e.attn_tune = (64, 4)
    e.attn_kind = "plain"
    import time
    e.started = time.monotonic()
    return e


def reference_rows(ref_root, cfg, w, prompt, dtype):
    e = reference_engine(ref_root, cfg, w, dtype)
    rows = []
    with torch.inference_mode():
        for t in range(1, len(prompt) + 1):
            ids = torch.tensor([prompt[:t]], dtype=torch.int64)
            e._ensure_shape(1, t, 1)
            rows.append(e._forward_prefill(ids, t)[0, -1].float())
    return torch.stack(rows)


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/the/reference/checkout")
    ref_root = sys.argv[1]
    out = {"note": "logits of alvinyuwen/starter engine/engine.py run on CPU in float32", "cases": []}
    tmp = tempfile.mkdtemp()
    for name, seed, length in CASES:
        # the reference has no window (tests/test_equivalence.py:57-60): switch it off for case C
        folder = make_folder(tmp, name, seed=seed, use_sliding_window=False, sliding_window=None)
        cfg, w = plain.read_model_folder(folder)
        prompt = random_prompt(length, cfg["vocab_size"], seed + 100)
        ref_logits = reference_rows(ref_root, cfg, w, prompt, torch.float32)
        mine = plain.plain_forward(cfg, w, prompt)
        print(name, "plain vs reference code: max abs diff", (mine - ref_logits).abs().max().item())
        ref_bf16 = reference_rows(ref_root, cfg, w, prompt, torch.bfloat16)
        w16 = {k: v.to(torch.bfloat16) for k, v in w.items()}
        mine16 = plain.plain_forward(cfg, w16, prompt)
        print(name, "the same in bfloat16: max abs diff", (mine16 - ref_bf16).abs().max().item(),
              "of max |logit|", ref_bf16.abs().max().item(),
              "; bfloat16 vs float32 reference:", (ref_bf16 - ref_logits).abs().max().item())
        out["cases"].append({
            "config": name, "seed": seed, "prompt": prompt,
            "overrides": {"use_sliding_window": False, "sliding_window": None},
            "logits": [[float(f"{v:.9g}") for v in row] for row in ref_logits.tolist()],
            "logits_bf16": [[float(f"{v:.5g}") for v in row] for row in ref_bf16.tolist()],
        })
    with open(os.path.join(HERE, "reference_logits.json"), "w") as handle:
        json.dump(out, handle, separators=(",", ":"))
    print("wrote", os.path.join(HERE, "reference_logits.json"))


if __name__ == "__main__":
    main()
