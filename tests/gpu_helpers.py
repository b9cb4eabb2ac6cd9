"""Shared pieces of the GPU tests: tolerances fixed in advance, model folders, comparison."""

import torch

import plain_qwen3 as plain
from tiny import make_folder, random_prompt

# All bounds are relative to the largest logit of the case (random N(0, 0.02) weights give logits of
# about 0.8 at the tiny sizes and 5 at real layer sizes), and were fixed from measurements of the
# engine and of the plain implementation itself on the tiny configurations and at real layer sizes.
#
# float32: both sides compute in 32-bit and differ only in the order of sums (measured: at most
# 6e-7 at the tiny sizes, 5.4e-6 with rows of 2,560 to 9,728 terms).
FP32_TOL = 2e-5
# bfloat16 against the float32 oracle.  The logits themselves are rounded to 8 bits of mantissa a
# handful of times per layer; the plain implementation run in bfloat16 differs from its float32 run
# by up to 1.4e-2 of the largest logit (mean 2.2e-3), the engine from the float32 oracle by up to
# 1.45e-2 (mean 2.3e-3), and two ways of cutting the same request differ by up to 1.1e-2 between
# themselves.  The largest error of a row may reach 2.5e-2; the mean error over a comparison, which
# is what a misplaced cast or a wrong key among hundreds moves, 4e-3.  (The reference accepts its
# own bfloat16 kernels at atol = rtol = 2e-2 per op, engine/engine.py:634, 977-979.)
BF16_TOL = 2.5e-2
BF16_MEAN_TOL = 4e-3

DTYPES = ["float32", "bfloat16"]


def tolerance(dtype, want):
    scale = float(want.abs().max())
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
    if dtype != "float32":
        mean = (got - want).abs().mean().item()
        bound = BF16_MEAN_TOL * float(want.abs().max())
        if not mean <= bound:
            raise AssertionError(f"{what}: mean error {mean:.3e} above {bound:.3e} although no row is "
                                 f"off by more than {tol:.2e}")


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
