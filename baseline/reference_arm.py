"""The reference arm of bench.py: alvinyuwen/starter's own engine, unmodified, on the same workload.

``baseline/_ref`` holds a plain copy of the reference's tree (it has no packaging metadata, so
there is nothing for pip to install).  Its ``engine/engine.py`` is imported from there as it is.
Only ``Engine.__init__`` is bypassed: it loads a checkpoint through a model library whose installed
version no longer has the attribute it reads (``config.rope_theta``, engine/engine.py:146), and the
benchmark runs random weights anyway.  The object is made with ``Engine.__new__`` and given what
``__init__`` would set (engine/engine.py:139-235): the sizes, random bfloat16 tensors of the Qwen3-4B
shapes with q/k/v and gate/up stacked, and its transposed weight copies.  Everything that computes is
the reference's own code on its own path: ``generate`` (engine/engine.py:1069-1105), hence
``_ensure_shape`` with kernel validation, attention and matmul selection, prefill selection and graph
capture (engine/engine.py:843-880), ``_forward_prefill`` and the captured ``_forward_decode``.  Which
of its kernels it adopted on this GPU is reported in the line (``reference_path``).

Nothing of starter_b200 (model, kernels, engine) is imported here.
"""

from __future__ import annotations

import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_ROOT = os.path.join(ROOT, "baseline", "_ref")


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def build_engine(ref, torch, sizes, seed=0):
    """An ``Engine`` of the reference with random weights, its ``__init__`` bypassed."""
    dev = ref.DEVICE
    gen = torch.Generator(device=dev).manual_seed(seed)
    dt = ref.LOAD_DTYPE

    def matrix(*shape):
        return (torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32) * 0.02).to(dt)

    def gain(n):
        return (1.0 + 0.1 * torch.randn(n, generator=gen, device=dev, dtype=torch.float32)).to(dt)

    torch.backends.cuda.matmul.allow_tf32 = False          # engine/engine.py:119-122
    torch.backends.cudnn.allow_tf32 = False
    e = ref.Engine.__new__(ref.Engine)
    e.started = time.monotonic()
    e.LAYERS = sizes["num_hidden_layers"]
    e.HIDDEN = sizes["hidden_size"]
    e.HEADS = sizes["num_attention_heads"]
    e.KV_HEADS = sizes["num_key_value_heads"]
    e.HEAD_DIM = sizes["head_dim"]
    e.GROUPS = e.HEADS // e.KV_HEADS
    e.EPS = sizes["rms_norm_eps"]
    e.THETA = sizes["rope_theta"]
    e.SCALE = e.HEAD_DIM ** -0.5
    q_size, kv_size, inter = e.HEADS * e.HEAD_DIM, e.KV_HEADS * e.HEAD_DIM, sizes["intermediate_size"]
    e.embed = matrix(sizes["vocab_size"], e.HIDDEN)
    e.final_norm_w = gain(e.HIDDEN)
    e.lm_head_w = e.embed if sizes["tie_word_embeddings"] else matrix(sizes["vocab_size"], e.HIDDEN)
    e.layers = []
    for idx in range(e.LAYERS):
        e.layers.append({
            "idx": idx, "in_ln": gain(e.HIDDEN), "qkv": matrix(q_size + 2 * kv_size, e.HIDDEN),
            "q_norm": gain(e.HEAD_DIM), "k_norm": gain(e.HEAD_DIM), "o": matrix(e.HIDDEN, q_size),
            "post_ln": gain(e.HIDDEN), "gate_up": matrix(2 * inter, e.HIDDEN), "down": matrix(e.HIDDEN, inter),
        })
    e.transposed = {}                                        # engine/engine.py:183-197
    try:
        for layer in e.layers:
            for name in ("qkv", "o", "gate_up", "down"):
                weight = layer[name]
                e.transposed[weight.data_ptr()] = weight.t().contiguous()
        e.transposed[e.lm_head_w.data_ptr()] = e.lm_head_w.t().contiguous()
    except torch.cuda.OutOfMemoryError:
        e.transposed = {}
    torch.cuda.empty_cache()
    e.dtype = e.embed.dtype
    e.cuda = True
    e.q_size, e.kv_size = q_size, kv_size
    e.rope_len = 0
    e.cos_table = e.sin_table = None
    e._grow_rope(4096)
    e.cache_k = e.cache_v = None
    e.capacity = e.batch = 0
    e.graph = e.g_token = e.g_pos = e.g_out = e.g_arange = None
    e.gqa = None
    e.time_probe = 0
    e.fused_norm = e.fused_rope = e.fused_swiglu = e.fused_attn = False
    e.fused_add_norm = e.fused_kv_cache = e.fused_norm_rope = False
    e.gemm_blocks = None
    e.gemm_choice = {}
    e.prefill_fused = True
    e.attn_tune = (64, 4)
    e.attn_kind = "plain"
    return e


def path_taken(e, ref) -> dict:
    """Which of its own alternatives the reference settled on for the last shape it built."""
    return {
        "triton_kernels": "unavailable: " + str(ref._kernels_error)[:80] if ref._kernels_error is not None else "imported",
        "graph": e.graph is not None,
        "attention": (e.attn_kind + str(tuple(e.attn_tune))) if e.fused_attn else ("sdpa_gqa" if e.gqa else "sdpa_repeat_kv"),
        "fused": "".join(c for c, on in (("n", e.fused_norm), ("r", e.fused_rope), ("s", e.fused_swiglu),
                                         ("N", e.fused_norm_rope), ("a", e.fused_add_norm),
                                         ("k", e.fused_kv_cache)) if on),
        "matmuls_own": len(e.gemm_choice),
        "prefill_fused": bool(e.prefill_fused),
    }


def run(args, sizes, context, prompt_len, decode_at, config_block, clock_sampler, metric) -> int:
    if args.gpus != 1:
        print(f"bench.py measures one GPU (asked for {args.gpus})")
        return 2
    if not os.path.isfile(os.path.join(REF_ROOT, "engine", "engine.py")):
        return unavailable("baseline/_ref holds no copy of the reference (engine/engine.py); copy the "
                           "reference's tree there")
    try:
        import torch
    except Exception as exc:  # noqa: BLE001
        return unavailable(f"torch cannot be imported: {exc}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device is visible")
    sys.path.insert(0, os.path.join(REF_ROOT, "engine"))
    try:
        import engine as ref          # the reference's engine/engine.py, as it is
    except Exception as exc:  # noqa: BLE001
        return unavailable(f"the reference's engine/engine.py cannot be imported: {str(exc)[:200]}")
    if os.path.realpath(ref.__file__) != os.path.realpath(os.path.join(REF_ROOT, "engine", "engine.py")):
        return unavailable(f"'engine' resolved to {ref.__file__}, not to the reference's copy")

    warmup, steps = max(args.warmup, 3), max(args.steps, 1)
    vocab = sizes["vocab_size"]
    windows = []
    clock_sampler.start()
    e = build_engine(ref, torch, sizes)
    gen = torch.Generator().manual_seed(0)

    def prompts(batch, n):
        return torch.randint(0, vocab, (batch, n), generator=gen).tolist()

    def decode_point(batch):
        """(device ms per step, end-to-end tok/s) of the reference's decode at ``decode_at`` tokens."""
        e.started = time.monotonic()          # a fresh tuning budget, as a fresh process would have
        stream = e.generate(prompts(batch, decode_at), warmup + steps + 1)
        next(stream)                           # builds, validates, tunes, captures; runs the prompts
        for _ in range(warmup):
            next(stream)
        torch.cuda.synchronize()
        t0 = time.monotonic()
        for _ in range(steps):
            next(stream)                       # each yield has copied the step's ids to the host
        torch.cuda.synchronize()
        t1 = time.monotonic()
        windows.append((t0, t1))
        stream.close()
        e2e = batch * steps / (t1 - t0)
        # the same steps on the device alone: its captured step replayed from the same position,
        # as its own _time_decode does (engine/engine.py:292-342)
        with torch.inference_mode():
            e.g_pos.fill_(decode_at)
            for _ in range(3):
                e._decode_step()
            e.g_pos.fill_(decode_at)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = time.monotonic()
            start.record()
            for _ in range(steps):
                e._decode_step()
            stop.record()
            torch.cuda.synchronize()
            windows.append((t0, time.monotonic()))
        return start.elapsed_time(stop) / steps, e2e

    try:
        ms, e2e = decode_point(args.batch)
        taken = path_taken(e, ref)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                b_ms, _ = decode_point(b)
                points[f"decode_b{b}"] = round(b / b_ms * 1e3, 1)
        # one prompt of 2,048 tokens.  Building this shape would tune the decode step for it first;
        # that is of no use here, so its tuning budget is marked spent (it then keeps the first
        # candidate of each choice); the prompt path is still chosen by its own _select_prefill.
        e.started = time.monotonic() - ref.TUNE_BUDGET_S - 1.0
        ids = torch.tensor(prompts(1, prompt_len), dtype=torch.int64, device=ref.DEVICE)
        with torch.inference_mode():
            e._ensure_shape(1, prompt_len, 1)
            for _ in range(warmup):
                e._forward_prefill(ids, prompt_len)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = time.monotonic()
            start.record()
            for _ in range(5):
                e._forward_prefill(ids, prompt_len)
            stop.record()
            torch.cuda.synchronize()
            windows.append((t0, time.monotonic()))
        prefill_ms = start.elapsed_time(stop) / 5
        taken["prefill_fused_1x2048"] = bool(e.prefill_fused)
    except Exception as exc:  # noqa: BLE001
        clock_sampler.stop(windows)
        return unavailable(f"the reference's engine failed on this GPU: {type(exc).__name__}: {str(exc)[:300]}")

    line = {
        "impl": "reference",
        "metric": metric,
        "value": round(args.batch / ms * 1e3, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": config_block,
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 8 * args.batch},
        "prefill": {"value": round(prompt_len / prefill_ms * 1e3, 1), "tokens": prompt_len,
                    "ms": round(prefill_ms, 3)},
        "points": points,
        "init": "bypassed: config.rope_theta (engine/engine.py:146); random weights set as __init__ would",
        "reference_path": taken,
        "clocks": clock_sampler.stop(windows),
    }
    print(json.dumps(line))
    return 0
