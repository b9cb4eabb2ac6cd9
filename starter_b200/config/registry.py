"""One registry from an architecture's name (``config.json["architectures"][0]``) to its model.

An entry is the architecture's typed config class; the class reads its own
``config.json`` keys and turns them into a ``ModelSpec`` from which the generic
decoder is built.  Adding an architecture is one ``register_architecture`` call.
"""

from __future__ import annotations

import json
import os

from .qwen3 import ConfigError, Qwen3Config

ARCHITECTURES: dict = {}


def register_architecture(name: str, config_cls) -> None:
    """``config_cls`` needs ``from_dict(raw)``, ``to_dict()`` and ``to_model_spec()``."""
    if name in ARCHITECTURES and ARCHITECTURES[name] is not config_cls:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = config_cls


register_architecture(Qwen3Config.architecture, Qwen3Config)


def config_from_dict(raw: dict):
    names = raw.get("architectures")
    if not names:
        raise ConfigError("config.json lacks required key(s): architectures")
    name = names[0]
    if name not in ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture {name!r}; known: " + ", ".join(sorted(ARCHITECTURES))
        )
    return ARCHITECTURES[name].from_dict(raw)


def load_config(model_dir: str):
    """Read ``model_dir/config.json`` and return the typed config its architecture names."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    with open(path, "r", encoding="utf-8") as handle:
        return config_from_dict(json.load(handle))
