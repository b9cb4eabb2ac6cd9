"""Decode and prefill throughput of starter_b200 at Qwen3-4B size on ONE B200, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints one JSON line.  A "step" is one decode step of the whole batch.  ``value`` is decoded
tokens per second at batch 8, timed on the device with CUDA events around K consecutive steps of
the captured, self-feeding decode step at the middle of the generation range (context 3,072 of
4,096); ``e2e`` is the same through ``Engine.generate``: host ids out every step, the host-owned inputs
of every step in from pinned memory, a step launched before the one before it is read;
``prefill`` is one 2,048-token prompt; ``points`` are decode at batch 1 and 64; ``roofline`` sets the
bytes a decode step must read (every weight it uses once, the live requests' keys and values)
against the measured copy bandwidth.  Every step reads >8 GB of weights, far more than the 126 MB
L2, so nothing is flushed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = dict(
    architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=2560, num_attention_heads=32,
    num_key_value_heads=8, head_dim=128, intermediate_size=9728, vocab_size=151936, rope_theta=5e6,
    rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096,
)
QWEN3_8B = dict(QWEN3_4B, hidden_size=4096, intermediate_size=12288, rope_theta=1e6, tie_word_embeddings=False)
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
#: the further rows of the measurement table: model sizes, and the generation workload quoted for each
WORKLOADS = {
    "8b": dict(config=QWEN3_8B, name="Qwen3-8B", batch=8, prompt_range=(512, 2048), new_tokens=256),
    "14b": dict(config=QWEN3_14B, name="Qwen3-14B", batch=32, prompt_range=(1024, 1024), new_tokens=512),
}
CONTEXT = 4096
PROMPT = 2048
DECODE_AT = 3072  # 2,048 prompt tokens + 1,024 decoded: the middle of the generation range


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            out["hbm_gbs"] = float(raw.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(raw.get("bf16_tflops", out["bf16_tflops"]))
            out["bf16_tflops_sustained"] = float(raw.get("bf16_tflops_sustained", out["bf16_tflops_sustained"]))
            out["source"] = "measured"
        except Exception:  # noqa: BLE001
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.monotonic(), line.strip()))

    def stop(self, windows):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for stamp, line in self.samples:
            if not any(a <= stamp <= b for a, b in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                clocks.append(int(parts[0]))
                max_clock = int(parts[1])
            except (ValueError, IndexError):
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


METRIC = "decode tok/s at batch 8 (Qwen3-4B BF16); prefill tok/s at 2,048 tokens; batch 1/64 in points"


def config_block(layers: int, batch: int, peaks_source: str) -> dict:
    """Every size of the run, flat; the same for both arms."""
    c = QWEN3_4B
    return {
        "model": "Qwen3-4B", "layers": layers, "layers_of_model": c["num_hidden_layers"],
        "hidden": c["hidden_size"], "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
        "head_dim": c["head_dim"], "intermediate": c["intermediate_size"], "vocab": c["vocab_size"],
        "tied": True, "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT,
        "decode_context": DECODE_AT, "parallelism": "single", "l2": "inputs larger than L2",
        "cache_page": 64, "peaks": peaks_source,
    }


def reference_arm(args) -> int:
    """The reference's own engine on the same workload (baseline/reference_arm.py)."""
    from baseline import reference_arm as arm

    sizes = dict(QWEN3_4B, num_hidden_layers=args.layers)
    return arm.run(args, sizes, CONTEXT, PROMPT, DECODE_AT,
                   config_block(args.layers, args.batch, peaks()["source"]), ClockSampler(), METRIC)


def per_stage(model, runner, slots, batch, peak_gbs, out=sys.stderr):
    """Where a decode step's time goes: every kind of kernel of a layer alone, in a CUDA graph that
    runs it once per layer on that layer's own weights and cache (so nothing stays in L2 from one
    launch to the next), timed with CUDA events; against the time its bytes take at the copy peak."""
    import torch

    from starter_b200 import ops

    spec = model.spec
    dev = model.device
    blocks = [model.blocks[e.layer] for e in spec.schedule]
    entries = [e.cache for e in spec.schedule]
    mixer = blocks[0].mixer.spec
    h = spec.hidden_size
    x = (torch.randn(batch, h, device=dev) * 0.5).to(torch.bfloat16)
    res = x.clone()
    attn_in = (torch.randn(batch, mixer.num_heads * mixer.head_dim, device=dev) * 0.5).to(torch.bfloat16)
    act = (torch.randn(batch, blocks[0].feed_forward.down.shape[1], device=dev) * 0.5).to(torch.bfloat16)
    qkv = (torch.randn(batch, blocks[0].mixer.qkv.shape[0], device=dev) * 0.5).to(torch.bfloat16)
    cache = runner.cache
    seq_slot = torch.tensor(slots, dtype=torch.int32, device=dev)
    kv_len = torch.tensor([cache.lengths[s] for s in slots], dtype=torch.int32, device=dev)
    kv_tokens = max(cache.lengths[s] for s in slots)
    rot = blocks[0].mixer.position.rotation()

    def attention(b, entry):
        keys, values = cache.entry_pages(entry)
        m = b.mixer
        return ops.attention_decode_qkv(qkv, keys, values, cache.block_table, seq_slot, kv_len, mixer.num_heads,
                                        mixer.num_kv_heads, mixer.head_dim, mixer.scale, mixer.window, m.q_norm,
                                        m.k_norm, mixer.qk_norm_eps, rot.cos, rot.sin, write_cache=True,
                                        kv_hint=kv_tokens, early=True)

    nbytes = lambda t: t.numel() * t.element_size()
    kv_bytes = cache.bytes_per_token() // len(set(entries)) * int(kv_len.sum())
    stages = [
        ("sum + norm (x2 per layer)", lambda b, e: ops.rmsnorm(res, b.norm1.weight, b.norm1.spec.eps, delta=x), lambda b: 0),
        ("q/k/v projection", lambda b, e: ops.linear(x, b.mixer.qkv), lambda b: nbytes(b.mixer.qkv)),
        ("attention (norm, rotation, cache write inside)", attention, lambda b: kv_bytes),
        ("output projection", lambda b, e: ops.linear(attn_in, b.mixer.o), lambda b: nbytes(b.mixer.o)),
        ("gate/up projection + SwiGLU", lambda b, e: ops.linear(x, b.feed_forward.gate_up, gated=True),
         lambda b: nbytes(b.feed_forward.gate_up)),
        ("down projection", lambda b, e: ops.linear(act, b.feed_forward.down), lambda b: nbytes(b.feed_forward.down)),
    ]
    rows, total = [], 0.0
    for name, fn, bytes_of in stages:
        for b, e in zip(blocks, entries):
            fn(b, e)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for b, e in zip(blocks, entries):
                fn(b, e)
        graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(5):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(stop) / 5 / len(blocks) * 1e3
        ideal = bytes_of(blocks[0]) / (peak_gbs * 1e9) * 1e6
        per_layer = us * (2 if name.startswith("sum") else 1)
        total += per_layer
        rows.append((name, us, ideal))
    print(f"decode step at batch {batch}, {kv_tokens} cached tokens per sequence: microseconds per launch, "
          f"inside a CUDA graph", file=out)
    for name, us, ideal in rows:
        frac = f"{ideal / us:.2f}" if ideal else "-"
        print(f"  {name:48s} {us:7.1f} us   bytes at {peak_gbs:.0f} GB/s: {ideal:6.1f} us   fraction {frac}", file=out)
    print(f"  a layer's seven launches one by one: {total:.1f} us", file=out)
    return total


def workload(args) -> int:
    """One of the further rows (``--workload 8b|14b``): a batch of prompts generated to the end through
    ``Engine.generate``, timed by the wall clock with the device idle on both sides.  Prints one JSON
    line: the whole job's generated tokens a second, the time to the first token (all prompts in one
    step), decode tokens a second after it, and the decode's share of its own memory roofline."""
    import torch

    from starter_b200.config import config_from_dict
    from starter_b200.engine import random_model
    from starter_b200.engine.entry import Engine

    spec = WORKLOADS[args.workload]
    raw = dict(spec["config"])
    layers_of_model = raw["num_hidden_layers"]
    raw["num_hidden_layers"] = min(args.layers, layers_of_model) if args.layers_given else layers_of_model
    config = config_from_dict(raw)
    model = random_model(config, seed=0, dtype="bfloat16")
    pk = peaks()
    gen = torch.Generator().manual_seed(0)
    lo, hi = spec["prompt_range"]
    lengths = [int(torch.randint(lo, hi + 1, (1,), generator=gen)) for _ in range(spec["batch"])]
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    new = spec["new_tokens"]
    engine = Engine.from_model(model, max_batch=spec["batch"])
    sampler = ClockSampler()
    sampler.start()
    for _ in engine.generate(prompts, 4):        # builds the cache, compiles, captures the first graphs
        pass
    best = None
    for _ in range(2):
        torch.cuda.synchronize()
        t0 = time.monotonic()
        stream = engine.generate(prompts, new)
        next(stream)
        torch.cuda.synchronize()
        t1 = time.monotonic()
        for _ in stream:
            pass
        torch.cuda.synchronize()
        t2 = time.monotonic()
        if best is None or t2 - t0 < best[2] - best[0]:
            best = (t0, t1, t2)
    t0, t1, t2 = best
    engine.runner.check_status()
    batch = spec["batch"]
    decode_ms = (t2 - t1) / (new - 1) * 1e3
    mean_context = sum(lengths) / batch + new / 2
    step_bytes = model.step_weight_bytes() + engine.runner.cache.bytes_per_token() * batch * mean_context
    achieved = step_bytes / (decode_ms * 1e-3) / 1e9
    line = {
        "metric": f"generated tok/s of the whole job ({spec['name']} BF16): {batch} prompts of {lo}-{hi} tokens, {new} new tokens each",
        "value": round(batch * new / (t2 - t0), 1), "unit": "tok/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": spec["name"], "layers": raw["num_hidden_layers"], "layers_of_model": layers_of_model,
                   "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
                   "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
                   "tied": raw["tie_word_embeddings"], "global_batch": batch, "prompt_tokens": sum(lengths),
                   "new_tokens": new, "peaks": pk["source"]},
        "ttft_ms": round((t1 - t0) * 1e3, 2),
        "prefill_tok_s": round(sum(lengths) / (t1 - t0), 1),
        "decode_tok_s": round(batch / decode_ms * 1e3, 1), "decode_ms_per_step": round(decode_ms, 4),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": sampler.stop([(t0, t2)]),
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=QWEN3_4B["num_hidden_layers"],
                        help="fewer layers than the model has (both numbers are reported)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                        help="instead of the default run: one of the further rows (other model sizes)")
    parser.add_argument("--decode-at", type=int, default=DECODE_AT,
                        help="cached tokens per sequence at which decode is timed (default: the middle of the "
                             "generation range); the cache is sized for it")
    parser.add_argument("--per-stage", action="store_true",
                        help="also print where a decode step's time goes, kernel by kernel (stderr)")
    args = parser.parse_args()
    args.layers_given = "--layers" in sys.argv
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (asked for {args.gpus})")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload:
        return workload(args)
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    decode_at = args.decode_at
    context = max(CONTEXT, -(-(decode_at + warmup + 2 * steps + 2) // 64) * 64)     # whole cache pages

    import torch

    from starter_b200 import ops
    from starter_b200.config import config_from_dict
    from starter_b200.engine import ModelRunner, StepEntry, random_model
    from starter_b200.engine.entry import Engine

    raw = dict(QWEN3_4B, num_hidden_layers=args.layers)
    config = config_from_dict(raw)
    model = random_model(config, seed=0, dtype="bfloat16")
    vocab = config.vocab_size
    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    windows = []
    gen = torch.Generator().manual_seed(0)

    def prompt(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    max_batch = max(args.batch, 1 if args.skip_points else 64)
    runner = ModelRunner(model, max_tokens=max_batch * context, max_sequences=max_batch)

    def timed(fn, reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.monotonic()
        start.record()
        for _ in range(reps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        windows.append((t0, time.monotonic()))
        return start.elapsed_time(stop) / reps

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    def prefill_once():
        slot = runner.open_sequence()
        runner.step([StepEntry(slot, prefill_prompt, [PROMPT - 1])])
        runner.close_sequence(slot)

    prefill_prompt = prompt(PROMPT)
    for _ in range(warmup):
        prefill_once()
    prefill_ms = timed(prefill_once, 5)
    h, nh, kv, d, inter, layers = (config.hidden_size, config.num_attention_heads,
                                   config.num_key_value_heads, config.head_dim,
                                   config.intermediate_size, args.layers)
    per_token = 2 * h * (nh + 2 * kv) * d + 2 * nh * d * h + 2 * h * 2 * inter + 2 * inter * h
    attn = 4 * nh * d * PROMPT * (PROMPT + 1) / 2
    prefill_flops = layers * (per_token * PROMPT + attn) + 2 * h * vocab
    prefill = {"value": round(PROMPT / prefill_ms * 1e3, 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               # the same against the vendor GEMM's throughput in a seconds-long loop under the power
               # cap: the prompt step is timed over several back-to-back repetitions
               "frac_of_sustained": round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}

    # ---------------------------------------------------------------- decode, device-timed
    def decode_point(batch):
        slots = [runner.open_sequence() for _ in range(batch)]
        for s in slots:
            runner.reserve(s, context)
            runner.step([StepEntry(s, prompt(decode_at), [])])
        entries = [StepEntry(s, [1], [0]) for s in slots]
        zeros = [0.0] * batch
        keys = [0] * batch

        def one():
            runner.decode_tokens(entries, zeros, keys)

        for _ in range(warmup):
            one()
        if args.per_stage:
            per_layer_us = per_stage(model, runner, slots, batch, pk["hbm_gbs"])
            one()
        before = ops.launch_count
        captured = len(runner.graphs.graphs)
        ms = timed(one, steps)
        if len(runner.graphs.graphs) != captured:
            # the sequences grew into the next length class inside the timed steps and its graph was
            # captured there: that is set-up, not a decode step; time the same number of steps again
            before = ops.launch_count
            ms = timed(one, steps)
        if args.per_stage:
            print(f"  the whole step: {ms * 1e3:.1f} us = {len(model.spec.schedule)} layers x "
                  f"{(ms * 1e3) / len(model.spec.schedule):.1f} us (head, sampling and embedding included); "
                  f"launched one by one the layers' kernels add up to {per_layer_us:.1f} us a layer",
                  file=sys.stderr)
        per_graph = runner.graphs.kernels_per_replay.get(batch, 0)
        launches = steps * per_graph + (ops.launch_count - before)
        for s in slots:
            runner.close_sequence(s)
        kv_bytes = runner.cache.bytes_per_token() * batch * (decode_at + warmup + steps / 2)
        return ms, launches, model.step_weight_bytes() + kv_bytes

    ms, launches, step_bytes = decode_point(args.batch)
    value = args.batch / ms * 1e3
    achieved = step_bytes / (ms * 1e-3) / 1e9
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            b_ms, _, _ = decode_point(b)
            points[f"decode_b{b}"] = round(b / b_ms * 1e3, 1)

    # ---------------------------------------------------------------- end to end through Engine.generate
    del runner
    torch.cuda.empty_cache()

    def e2e_point(batch):
        """tok/s through the public call: prompts in as host lists, one list of ids out per step."""
        engine = Engine.from_model(model, max_batch=batch)
        stream = engine.generate([prompt(decode_at) for _ in range(batch)], warmup + steps + 2)
        next(stream)
        # every step's host-owned inputs (positions, slots, lengths, sampling settings) travel from
        # pinned host memory to the device and the drawn ids travel back to the host; the ids a step
        # consumes are the ones the step before drew on the device, so the loop launches a step
        # before it reads the one before (one step of lookahead, as the reference's loop does)
        engine.runner.self_feeding = False
        for _ in range(warmup):
            next(stream)
        torch.cuda.synchronize()
        t0 = time.monotonic()
        for _ in range(steps):
            next(stream)
        torch.cuda.synchronize()
        t1 = time.monotonic()
        windows.append((t0, t1))
        stream.close()
        engine.runner.check_status()
        del engine
        torch.cuda.empty_cache()
        return batch * steps / (t1 - t0)

    e2e_value = e2e_point(args.batch)
    if not args.skip_points:
        points["e2e_b1"] = round(e2e_point(1), 1)

    clocks = sampler.stop(windows)
    line = {
        "metric": METRIC,
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": dict(config_block(args.layers, args.batch, pk["source"]), decode_context=decode_at),
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": 5 * 4 * args.batch,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
