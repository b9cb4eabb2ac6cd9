"""Trace replay: feeds given token ids through a model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
    python -m starter_b200 replay --model DIR --dtype ... --out DIR --max-tokens N

Reads one JSON object per line from standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

runs exactly those tokens through the library's own model, step function, cache and kernels (the
ones generation uses), writes ``OUT/<step>.f32`` (little-endian float32 ``[wanted, vocab]``, in the
order of the entries and of ``want``) when something is wanted, releases what the requests in ``end``
hold, and prints ``done <step>``.  It samples nothing.  ``--max-tokens`` sizes the cache: the most
tokens live requests hold at any time, each request rounded up to 64 (the cache's page).

The reference has no such program; its nearest idea is the platform's teacher-forced replay of the
emitted tokens (QWEN_ENGINE_CONTRACT.md:105-123).
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True)
    parser.add_argument("--max-tokens", type=int, required=True)
    args = parser.parse_args(argv)

    print("[trace_run] starting (the first call compiles the kernels this model needs)",
          file=sys.stderr, flush=True)
    from .cache.layout import PAGE_TOKENS, pages_for
    from .engine import ModelRunner, StepEntry, load_model

    os.makedirs(args.out, exist_ok=True)
    model = load_model(args.model, args.dtype)
    pages = max(pages_for(args.max_tokens), 1)
    runner = ModelRunner(model, pages * PAGE_TOKENS, max_sequences=min(pages, 4096), use_graphs=False)
    print(f"[trace_run] model loaded; cache of {pages} pages of {PAGE_TOKENS} tokens", file=sys.stderr,
          flush=True)

    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            rid = item["id"]
            if rid not in slots:
                slots[rid] = runner.open_sequence()
            entries.append(StepEntry(slots[rid], [int(t) for t in item["tokens"]],
                                     [int(w) for w in item.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                data = logits.to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                data.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            runner.check_status()
        for rid in record.get("end", []):
            if rid in slots:
                runner.close_sequence(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0
