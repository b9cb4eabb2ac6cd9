"""Shared pieces of the GPU tests: tolerances fixed in advance, model folders, comparison."""

import torch

import plain_qwen3 as plain
from tiny import make_folder, random_prompt

# float32: both sides compute in 32-bit and differ only in the order of sums.
FP32_TOL = 2e-5
# bfloat16 against the float32 oracle: 8 bits of mantissa per rounding, a handful of roundings per
# layer; the reference accepts its own bfloat16 kernels at atol = rtol = 2e-2 per op
# (engine/engine.py:634, 977-979).  Relative to the largest logit of the case.
BF16_TOL = 3e-2

DTYPES = ["float32", "bfloat16"]


def tolerance(dtype, want):
    scale = max(1.0, float(want.abs().max()))
    return (FP32_TOL if dtype == "float32" else BF16_TOL) * scale


def assert_close(got, want, dtype, what=""):
    """Fails with the first wrong row named: its place is the clue (a prompt's end, the first
    single-token step, a page boundary)."""
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    tol = tolerance(dtype, want)
    err = (got - want).abs().reshape(want.shape[0], -1).max(dim=1).values
    bad = (~(err <= tol)).nonzero().flatten().tolist()
    if bad:
        raise AssertionError(f"{what}: {len(bad)} of {len(err)} rows off by more than {tol:.2e}; "
                             f"first wrong row {bad[0]} (error {err[bad[0]].item():.3e}), "
                             f"largest error {err.max().item():.3e}")


_cache = {}


def model_case(tmp_path_factory, name, seed=1):
    """(folder, config dict, float32 weights) of a tiny random model, made once per session."""
    key = (name, seed)
    if key not in _cache:
        folder = make_folder(tmp_path_factory.mktemp(f"m{name}{seed}"), name, seed=seed)
        cfg, w = plain.read_model_folder(folder)
        _cache[key] = (folder, cfg, w)
    return _cache[key]


_runners = {}


def runner_for(tmp_path_factory, name, dtype, max_tokens=64 * 48, seed=1):
    from starter_b200.engine import ModelRunner, load_model

    key = (name, dtype, max_tokens, seed)
    if key not in _runners:
        folder, _, _ = model_case(tmp_path_factory, name, seed)
        _runners[key] = ModelRunner(load_model(folder, dtype), max_tokens=max_tokens, max_sequences=16)
    return _runners[key]
