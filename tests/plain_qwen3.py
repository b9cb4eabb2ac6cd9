"""A plain, slow statement of the Qwen3 dense decoder: whole sequences, no cache, one function per part.

Written from the reference's formulas (each function cites them) and sharing no
code with ``starter_b200``: it reads ``config.json`` and ``model.safetensors`` with
the ``json`` module and the ``safetensors`` package and computes with torch on the
CPU.  ``dtype`` float32 is the oracle; with bfloat16 the casts fall where the
reference places them, since the formulas are written in the reference's order.

Compared once with the reference's own forward code on tiny random models: see
tests/golden/make_golden.py and tests/test_plain.py::test_plain_matches_reference_code.
The window rule, temperature sampling and unequal batches are not in the reference;
they rest on the formulas stated here.
"""

from __future__ import annotations

import json
import math
import os

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- loading

def read_model_folder(path, dtype=torch.float32):
    """``(config dict, {name: tensor})`` with every tensor cast to ``dtype``."""
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as handle:
        cfg = json.load(handle)
    weights = {k: v.to(dtype) for k, v in load_file(os.path.join(path, "model.safetensors")).items()}
    return cfg, weights


def head_dim_of(cfg):
    # engine/engine.py:143
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_window(cfg, layer):
    """None, or the window of this layer (not in the reference, whose model has none:
    tests/test_equivalence.py:57-60).  Layers from ``max_window_layers`` on are windowed."""
    if not cfg.get("use_sliding_window") or cfg.get("sliding_window") is None:
        return None
    return cfg["sliding_window"] if layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"]) else None


# --------------------------------------------------------------------------- parts

def plain_rms_norm(x, weight, eps):
    """engine/engine.py:75-88: reduce and scale in float32, cast to the input dtype, then the gain."""
    dtype = x.dtype
    xf = x.float()
    variance = xf.pow(2).mean(-1, keepdim=True)
    xf = xf * torch.rsqrt(variance + eps)
    return weight * xf.to(dtype)


def plain_rope_tables(theta, head_dim, length, dtype):
    """engine/engine.py:240-259: float32 angles, ``cat(freqs, freqs)``, cast once."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim
    inv_freq = 1.0 / (theta ** exponent)
    pos = torch.arange(length, dtype=torch.int64).float()
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def plain_rotate_half(x):
    """engine/engine.py:91-93."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def plain_apply_rope(x, cos, sin):
    """engine/engine.py:96-109 on ``[T, heads, D]`` with tables ``[T, D]``."""
    cos = cos.unsqueeze(1)
    sin = sin.unsqueeze(1)
    return (x * cos) + (plain_rotate_half(x) * sin)


def plain_attention(q, k, v, scale, window=None):
    """Causal grouped-query attention of one whole sequence.

    q ``[T, heads, D]``, k and v ``[T, kv_heads, D]``.  Query head h uses key/value
    head ``h // (heads // kv_heads)`` (engine/engine.py:276-277); scores are
    ``q.k * scale`` (engine/engine.py:147, 272-280); key j is visible to query i iff
    ``j <= i`` (engine/engine.py:783-785) and, with a window w, ``j > i - w``; softmax
    over keys in float32; output ``P.V``.
    """
    tokens, heads, _ = q.shape
    groups = heads // k.shape[1]
    kx = k.repeat_interleave(groups, dim=1)
    vx = v.repeat_interleave(groups, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q.float(), kx.float()) * scale
    i = torch.arange(tokens).unsqueeze(1)
    j = torch.arange(tokens).unsqueeze(0)
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    scores = scores.masked_fill(~visible.unsqueeze(0), float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", probs, vx.float())
    return out.to(q.dtype)


def plain_swiglu(gate, up):
    """engine/engine.py:464-468: ``silu(gate) * up``; silu's result is in the working dtype."""
    return F.silu(gate) * up


def plain_mixer(n, w, prefix, cfg, cos, sin, window):
    """The attention part of engine/engine.py:679-734: q/k/v projections without bias, per-head
    RMSNorm of q and k over head_dim with the model's eps, rotation, attention, output projection."""
    heads, kv_heads, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    tokens = n.shape[0]
    q = F.linear(n, w[prefix + "self_attn.q_proj.weight"]).view(tokens, heads, d)
    k = F.linear(n, w[prefix + "self_attn.k_proj.weight"]).view(tokens, kv_heads, d)
    v = F.linear(n, w[prefix + "self_attn.v_proj.weight"]).view(tokens, kv_heads, d)
    if cfg.get("qk_norm", True):
        q = plain_rms_norm(q, w[prefix + "self_attn.q_norm.weight"], cfg["rms_norm_eps"])
        k = plain_rms_norm(k, w[prefix + "self_attn.k_norm.weight"], cfg["rms_norm_eps"])
    q = plain_apply_rope(q, cos, sin)
    k = plain_apply_rope(k, cos, sin)
    a = plain_attention(q, k, v, d ** -0.5, window)
    return F.linear(a.reshape(tokens, heads * d), w[prefix + "self_attn.o_proj.weight"])


def plain_feed_forward(m, w, prefix):
    """engine/engine.py:735."""
    gate = F.linear(m, w[prefix + "mlp.gate_proj.weight"])
    up = F.linear(m, w[prefix + "mlp.up_proj.weight"])
    return F.linear(plain_swiglu(gate, up), w[prefix + "mlp.down_proj.weight"])


def plain_block(x, w, layer, cfg, cos, sin):
    """engine/engine.py:665-736 without the fusion of sums and norms: pre-norm, two residual sums."""
    prefix = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    n = plain_rms_norm(x, w[prefix + "input_layernorm.weight"], eps)
    x = x + plain_mixer(n, w, prefix, cfg, cos, sin, layer_window(cfg, layer))
    m = plain_rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps)
    return x + plain_feed_forward(m, w, prefix)


def plain_forward(cfg, w, tokens):
    """Logits ``[T, vocab]`` (float32) at every position of one sequence (engine/engine.py:768-803:
    embedding without scaling, the layers, the final norm, the head; tied head = the embedding)."""
    ids = torch.as_tensor(tokens, dtype=torch.int64)
    embed = w["model.embed_tokens.weight"]
    x = F.embedding(ids, embed)
    cos, sin = plain_rope_tables(cfg["rope_theta"], head_dim_of(cfg), len(tokens), x.dtype)
    for layer in range(cfg["num_hidden_layers"]):
        x = plain_block(x, w, layer, cfg, cos, sin)
    h = plain_rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = embed if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return F.linear(h, head).float()


# --------------------------------------------------------------------------- token selection

def _mix32(x):
    x = np.asarray(x, dtype=np.uint32).copy()
    x ^= x >> np.uint32(16)
    x *= np.uint32(0x7FEB352D)
    x ^= x >> np.uint32(15)
    x *= np.uint32(0x846CA68B)
    x ^= x >> np.uint32(16)
    return x


def plain_gumbel(request_key, position, vocab):
    """The noise added to ``logits / temperature`` before the argmax (ours, not the reference's):
    ``-log(-log(u_i))``, ``u_i`` from a hash of (request key, position, i)."""
    with np.errstate(over="ignore"):
        row_key = _mix32(np.uint32(position) + _mix32(np.uint32(request_key)))
        r = _mix32(np.arange(vocab, dtype=np.uint32) ^ row_key)
    u = ((r >> np.uint32(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)


def plain_request_key(seed, request_index):
    with np.errstate(over="ignore"):
        return int(_mix32(np.uint32(request_index) + _mix32(np.uint32(seed & 0xFFFFFFFF))))


def plain_select(logits, temperature, request_key=0, position=0):
    """Greedy: lowest index among the maxima (engine/engine.py:833).  Else argmax of
    ``logits / temperature`` plus Gumbel noise, which draws from ``softmax(logits / temperature)``."""
    row = np.asarray(logits, dtype=np.float32)
    if temperature <= 0:
        return int(np.argmax(row))
    noisy = row * np.float32(1.0 / np.float32(temperature)) + plain_gumbel(request_key, position, row.size)
    return int(np.argmax(noisy))


def plain_generate(cfg, w, prompt, max_new_tokens, temperature=0.0, seed=0, request_index=0,
                   stop_tokens=()):
    """Re-run the whole sequence for every new token; returns the new tokens (stop token included)."""
    seq = list(prompt)
    out = []
    key = plain_request_key(seed, request_index)
    for _ in range(max_new_tokens):
        logits = plain_forward(cfg, w, seq)[-1].numpy()
        tok = plain_select(logits, temperature, key, len(seq))
        out.append(tok)
        seq.append(tok)
        if tok in stop_tokens:
            break
    return out
