"""Random weights from a configuration and a seed, as tensors or as a model folder on disk.

Matrices are N(0, 0.02); norm gains are 1 + N(0, 0.1).  Each tensor is drawn in
float32 from a generator of its own, seeded from the seed and the tensor's name,
so a tensor's values depend on nothing but (seed, name, shape) and the order of
generation does not matter.  (The reference's test draws N(0, 0.05) for every
parameter through its model library, tests/test_equivalence.py:62-68.)
"""

from __future__ import annotations

import json
import os
import zlib

import torch

from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
GAIN_STD = 0.1


def _generator(seed: int, name: str, device) -> torch.Generator:
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63 - 1))
    return gen


def random_tensor(seed: int, name: str, spec, dtype, device="cpu") -> torch.Tensor:
    gen = _generator(seed, name, device)
    values = torch.randn(tuple(spec.shape), generator=gen, dtype=torch.float32, device=device)
    if spec.role == "gain":
        values.mul_(GAIN_STD).add_(1.0)
    else:
        values.mul_(MATRIX_STD)
    return values.to(dtype)


def random_checkpoint(expected: dict, seed: int, dtype, device="cpu") -> dict:
    """``{name: tensor}`` for every expected name (values differ between CPU and CUDA generators)."""
    return {name: random_tensor(seed, name, spec, dtype, device) for name, spec in expected.items()}


def write_model_folder(path: str, config, seed: int, dtype=torch.float32) -> str:
    """Write ``config.json`` and ``model.safetensors`` with random weights; returns ``path``.

    ``config`` is a typed config (``to_dict``, ``to_model_spec``).  Tensors are drawn
    on the CPU one at a time while the file is written.
    """
    from ..engine.model import expected_tensors

    os.makedirs(path, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(raw, handle, indent=1, sort_keys=True)
    expected = expected_tensors(config.to_model_spec())
    layout = [(name, dtype, tuple(spec.shape)) for name, spec in expected.items()]
    write_safetensors(
        os.path.join(path, "model.safetensors"),
        (layout, lambda name: random_tensor(seed, name, expected[name], dtype)),
        metadata={"format": "pt", "seed": seed},
    )
    return path
