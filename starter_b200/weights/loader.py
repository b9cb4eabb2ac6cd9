"""Loads a model's tensors from safetensors by name, checks them against what the model expects,
and places them on the device.

Placement: matrices are kept in the working dtype (bfloat16 in serving, float32 on
the 32-bit path); integer tables become int32; a gain that the checkpoint stores
in 32-bit stays 32-bit.  Everything that is wrong with a checkpoint is reported in
ONE error that lists the missing tensors, the unexpected ones and the wrong
shapes.  The reference leaves all of this to ``from_pretrained``
(engine/engine.py:124-133); tensor names are those of engine/engine.py:149-180.
"""

from __future__ import annotations

from collections.abc import Mapping

import torch

from ..parts.base import role_of
from .safetensors_io import open_model_files


class WeightError(ValueError):
    """A checkpoint that does not fit the model; ``missing``, ``unexpected``, ``wrong_shape``, ``other``."""

    def __init__(self, missing, unexpected, wrong_shape, other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        for item in self.other:
            lines.append("  " + item)
        super().__init__("\n".join(lines))


def place(tensor: torch.Tensor, role: str, dtype, device) -> torch.Tensor:
    """Move one stored tensor to the device in the dtype its role calls for."""
    if not tensor.dtype.is_floating_point:
        return tensor.to(device=device, dtype=torch.int32)
    if role_of(role).keep_32bit and tensor.dtype in (torch.float32, torch.float64):
        return tensor.to(device=device, dtype=torch.float32)
    return tensor.to(device=device, dtype=dtype)


def check_names(expected: dict, stored: dict, optional=()):
    """Compare ``expected`` (name -> ParamSpec) with ``stored`` (name -> (dtype, shape))."""
    missing = [n for n in expected if n not in stored]
    unexpected = [n for n in stored if n not in expected and n not in optional]
    wrong = [(n, stored[n][1], tuple(expected[n].shape)) for n in expected
             if n in stored and tuple(stored[n][1]) != tuple(expected[n].shape)]
    other = [f"{n} is stored as {stored[n][0]}, not a floating-point type" for n in expected
             if n in stored and not stored[n][0].is_floating_point]
    return missing, unexpected, wrong, other


class CheckpointTensors(Mapping):
    """``tensors[name]`` reads one stored tensor and places it on the device, when it is asked for and
    not before: a model that stacks q/k/v and gate/up layer by layer then never holds much more than
    one copy of the weights (the reference fuses layer by layer for the same reason,
    engine/engine.py:157-165)."""

    def __init__(self, owners: dict, expected: dict, dtype, device):
        self._owners, self._expected, self._dtype, self._device = owners, expected, dtype, device

    def __iter__(self):
        return iter(self._expected)

    def __len__(self) -> int:
        return len(self._expected)

    def __getitem__(self, name):
        spec = self._expected[name]
        return place(self._owners[name].tensor(name), spec.role, self._dtype, self._device)

    def pop(self, name, default=None):
        """Nothing is kept, so there is nothing to let go of."""
        return default


def load_checkpoint(model_dir: str, expected: dict, dtype, device, tied_alias=None):
    """Check the checkpoint against ``expected`` and return a mapping ``name -> device tensor`` that
    reads and places each tensor when it is indexed.

    ``tied_alias = (alias, target)``: ``alias`` is not expected; if the checkpoint
    holds it anyway it must equal ``target`` exactly, else that is reported.
    """
    owners = open_model_files(model_dir)
    stored = {name: handle.entries[name] for name, handle in owners.items()}
    optional = (tied_alias[0],) if tied_alias else ()
    missing, unexpected, wrong, other = check_names(expected, stored, optional)
    if tied_alias and tied_alias[0] in stored and tied_alias[1] in stored and not (missing or wrong):
        alias, target = tied_alias
        a, b = owners[alias].tensor(alias), owners[target].tensor(target)
        if a.shape != b.shape or a.dtype != b.dtype or not torch.equal(a, b):
            other.append(f"{alias} is stored and differs from {target}, but the config ties them")
    if missing or unexpected or wrong or other:
        raise WeightError(missing, unexpected, wrong, other)
    return CheckpointTensors(owners, expected, dtype, device)
