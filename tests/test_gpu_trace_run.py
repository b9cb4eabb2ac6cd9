"""bin/trace_run as a user drives it: the same requests whole, with the last 32 tokens one by one,
and in batches of unequal lengths, in float32 and in bfloat16, against the plain implementation."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from gpu_helpers import DTYPES, assert_close, model_case
from tiny import random_prompt

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(folder, dtype, steps, out_dir, max_tokens):
    """Feed the steps one at a time, each only after ``done`` for the one before."""
    proc = subprocess.Popen([sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out",
                             out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for record in steps:
        proc.stdin.write(json.dumps(record) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {record['step']}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


def read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_whole_stepwise_and_batched(tmp_path_factory, tmp_path, name, dtype):
    folder, cfg, w = model_case(tmp_path_factory, name)
    vocab = cfg["vocab_size"]
    reqs = {rid: random_prompt(n, vocab, 400 + n) for rid, n in (("a", 70), ("b", 37), ("c", 130), ("d", 33))}
    want = {rid: plain.plain_forward(cfg, w, toks) for rid, toks in reqs.items()}

    # 1. each request alone and whole; every place wanted; 64-token rounding: 192 tokens at most live
    out1 = str(tmp_path / "whole")
    steps = [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
             for i, (rid, toks) in enumerate(reqs.items())]
    replay(folder, dtype, steps, out1, max_tokens=192)
    for i, rid in enumerate(reqs):
        assert_close(read(out1, i, vocab), want[rid], dtype, f"whole {rid}")

    # 2. the last 32 tokens one by one
    out2 = str(tmp_path / "tail")
    toks = reqs["a"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:38], "want": [37]}], "end": []}]
    for i in range(32):
        steps.append({"step": 1 + i, "entries": [{"id": "a", "tokens": [toks[38 + i]], "want": [0]}],
                      "end": ["a"] if i == 31 else []})
    replay(folder, dtype, steps, out2, max_tokens=128)
    got = torch.cat([read(out2, s, vocab) for s in range(33)])
    assert_close(got, want["a"][37:], dtype, "last 32 one by one")

    # 3. two batches of unequal lengths one after another; shorter requests end earlier; a step in
    #    which nothing is wanted writes no file
    out3 = str(tmp_path / "batched")
    heads = {"a": 60, "b": 30, "c": 125, "d": 33}
    steps, n = [], 0
    got = {rid: [] for rid in reqs}
    plan = []
    for batch in (["a", "b"], ["c", "d"]):
        steps.append({"step": n, "entries": [{"id": r, "tokens": reqs[r][:heads[r]], "want": [heads[r] - 1]}
                                             for r in batch], "end": [r for r in batch if heads[r] == len(reqs[r])]})
        plan.append((n, [(r, heads[r] - 1) for r in batch]))
        n += 1
        at = dict(heads)
        live = [r for r in batch if at[r] < len(reqs[r])]
        while live:
            wanted = n % 3 != 0
            steps.append({"step": n, "entries": [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0] if wanted else []}
                                                 for r in live], "end": [r for r in live if at[r] + 1 == len(reqs[r])]})
            plan.append((n, [(r, at[r]) for r in live] if wanted else []))
            for r in live:
                at[r] += 1
            live = [r for r in live if at[r] < len(reqs[r])]
            n += 1
    replay(folder, dtype, steps, out3, max_tokens=256)        # a: 128 + b: 64, then c: 192 + d: 64
    for step, places in plan:
        path = os.path.join(out3, f"{step}.f32")
        if not places:
            assert not os.path.exists(path)
            continue
        rows = read(out3, step, vocab)
        assert rows.shape[0] == len(places)
        for row, (r, place) in zip(rows, places):
            assert_close(row[None], want[r][place][None], dtype, f"batched {r} place {place}")


def test_command_line_generates_what_the_plain_implementation_generates(tmp_path_factory):
    folder, cfg, w = model_case(tmp_path_factory, "A")
    prompts = [random_prompt(5, cfg["vocab_size"], 1), random_prompt(3, cfg["vocab_size"], 2)]
    text = ";".join(",".join(str(t) for t in p) for p in prompts)
    out = subprocess.run([sys.executable, "-m", "starter_b200", "generate", "--model-path", folder,
                          "--input-ids", text, "--max-new-tokens", "4", "--dtype", "float32"],
                         cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    assert [l["tokens"] for l in lines] == [plain.plain_generate(cfg, w, p, 4) for p in prompts]
    assert all(l["finish_reason"] == "length" for l in lines)
    # random prompts by length, a temperature, a stop token
    out = subprocess.run([sys.executable, "-m", "starter_b200", "generate", "--model-path", folder,
                          "--prompt-lens", "7,2", "--prompt-seed", "9", "--max-new-tokens", "5", "--dtype",
                          "float32", "--temperature", "0.9", "--seed", "4"],
                         cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    draw = torch.Generator().manual_seed(9)
    drawn = [torch.randint(0, cfg["vocab_size"], (n,), generator=draw).tolist() for n in (7, 2)]
    assert [l["tokens"] for l in lines] == [plain.plain_generate(cfg, w, p, 5, 0.9, 4, i) for i, p in enumerate(drawn)]
