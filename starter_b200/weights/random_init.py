"""Random weights from a configuration and a seed, as tensors or as a model folder on disk.

Matrices are N(0, 0.02); norm gains are 1 + N(0, 0.1); every other kind of tensor is drawn as its
role says (``starter_b200.parts.base.ROLES``), and a role nobody registered is an error.  Each tensor is drawn in
float32 from a generator of its own, seeded from the seed and the tensor's name,
so a tensor's values depend on nothing but (seed, name, shape) and the order of
generation does not matter.  (The reference's test draws N(0, 0.05) for every
parameter through its model library, tests/test_equivalence.py:62-68.)
"""

from __future__ import annotations

import json
import os
import zlib
from collections.abc import Mapping

import torch

from ..parts.base import role_of
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device) -> torch.Generator:
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63 - 1))
    return gen


def random_tensor(seed: int, name: str, spec, dtype, device="cpu") -> torch.Tensor:
    gen = _generator(seed, name, device)
    values = torch.randn(tuple(spec.shape), generator=gen, dtype=torch.float32, device=device)
    role = role_of(spec.role)
    values.mul_(role.std).add_(role.mean)
    return values.to(dtype)


class RandomTensors(Mapping):
    """``tensors[name]`` draws that tensor when it is asked for (the same values every time: they
    depend on nothing but the seed, the name and the shape), so a model that takes its tensors layer
    by layer never holds more than it keeps."""

    def __init__(self, expected: dict, seed: int, dtype, device):
        self._expected, self._seed, self._dtype, self._device = expected, seed, dtype, device

    def __iter__(self):
        return iter(self._expected)

    def __len__(self) -> int:
        return len(self._expected)

    def __getitem__(self, name):
        return random_tensor(self._seed, name, self._expected[name], self._dtype, self._device)

    def pop(self, name, default=None):
        return default


def random_checkpoint(expected: dict, seed: int, dtype, device="cpu") -> RandomTensors:
    """A mapping ``name -> tensor`` over every expected name (values differ between CPU and CUDA
    generators)."""
    return RandomTensors(expected, seed, dtype, device)


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
