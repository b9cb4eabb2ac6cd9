"""Configuration of the Qwen3 dense decoder, read from the keys of its own ``config.json``.

The reference engine copies ``num_hidden_layers``, ``hidden_size``,
``num_attention_heads``, ``num_key_value_heads``, ``head_dim`` (falling back to
``hidden_size // num_attention_heads``), ``rms_norm_eps`` and ``rope_theta`` off
the loaded checkpoint's config (engine/engine.py:139-147) and fixes the rest in
code: scale ``head_dim ** -0.5`` (engine/engine.py:147), SiLU gating
(engine/engine.py:464-468), no biases, per-head q/k norms always on
(engine/engine.py:699-708), no sliding window (tests/test_equivalence.py:57-60).
Here every one of those is a field, a key that asks for something this
architecture's parts cannot do is an error, and nothing is silently ignored.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Optional

from .spec import (
    AttentionSpec,
    GatedFeedForwardSpec,
    prenorm_layer,
    ModelSpec,
    NormSpec,
    RopeSpec,
    default_schedule,
)


class ConfigError(ValueError):
    """A config.json that is incomplete or asks for something unsupported."""


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "num_key_value_heads",
    "rms_norm_eps",
)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    hidden_act: str
    qk_norm: bool
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    torch_dtype: str

    architecture = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in raw]
        rope_theta = raw.get("rope_theta")
        if rope_theta is None and isinstance(raw.get("rope_parameters"), dict):
            rope_theta = raw["rope_parameters"].get("rope_theta")
        if rope_theta is None:
            missing.append("rope_theta")
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))

        def unsupported(key, value, why):
            raise ConfigError(f"config.json has {key}={value!r}: {why}")

        scaling = raw.get("rope_scaling")
        if scaling not in (None, {}):
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                unsupported("rope_scaling", scaling, "only unscaled rotary positions are implemented")
        params = raw.get("rope_parameters")
        if isinstance(params, dict) and params.get("rope_type", "default") != "default":
            unsupported("rope_parameters", params, "only unscaled rotary positions are implemented")
        if raw.get("attention_bias", False):
            unsupported("attention_bias", True, "the projections of this architecture have no bias")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            unsupported("hidden_act", act, "the gated feed-forward implements silu only")
        if raw.get("attention_dropout", 0.0):
            unsupported("attention_dropout", raw["attention_dropout"], "inference has no dropout")

        heads = int(raw["num_attention_heads"])
        kv_heads = int(raw["num_key_value_heads"])
        hidden = int(raw["hidden_size"])
        layers = int(raw["num_hidden_layers"])
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"head_dim is absent and hidden_size={hidden} is not a multiple of "
                    f"num_attention_heads={heads}"
                )
            head_dim = hidden // heads
        head_dim = int(head_dim)
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads={heads} must be a positive multiple of num_key_value_heads={kv_heads}"
            )
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"head_dim={head_dim} must be even for half-split rotary positions")
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers"):
            if int(raw[key]) <= 0:
                raise ConfigError(f"{key}={raw[key]} must be positive")
        eps = float(raw["rms_norm_eps"])
        if not eps > 0.0:
            raise ConfigError(f"rms_norm_eps={eps} must be positive")

        use_window = bool(raw.get("use_sliding_window", False))
        window = raw.get("sliding_window")
        if use_window:
            if window is None or int(window) <= 0:
                raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")
            window = int(window)
        else:
            window = None
        max_window_layers = int(raw.get("max_window_layers", layers))

        cfg = cls(
            vocab_size=int(raw["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=eps,
            rope_theta=float(rope_theta),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 0)),
            hidden_act=act,
            qk_norm=bool(raw.get("qk_norm", True)),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=max_window_layers,
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )
        types = raw.get("layer_types")
        if types is not None:
            want = [("sliding_attention" if w is not None else "full_attention") for w in cfg.layer_windows()]
            if list(types) != want:
                raise ConfigError(
                    "layer_types disagrees with use_sliding_window/sliding_window/max_window_layers: "
                    f"{list(types)} vs {want}"
                )
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as handle:
            return cls.from_dict(json.load(handle))

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        out = asdict(self)
        out["architectures"] = [self.architecture]
        out["model_type"] = "qwen3"
        out["attention_bias"] = False
        return out

    # ------------------------------------------------------------------ meaning

    def layer_windows(self) -> list:
        """The window of each layer: the first ``max_window_layers`` layers see all keys."""
        if not self.use_sliding_window:
            return [None] * self.num_hidden_layers
        return [
            None if i < self.max_window_layers else self.sliding_window
            for i in range(self.num_hidden_layers)
        ]

    def to_model_spec(self) -> ModelSpec:
        rope = RopeSpec(head_dim=self.head_dim, theta=self.rope_theta)
        ff = GatedFeedForwardSpec(
            hidden_size=self.hidden_size,
            intermediate_size=self.intermediate_size,
            activation=self.hidden_act,
        )
        norm = NormSpec(size=self.hidden_size, eps=self.rms_norm_eps)
        layers = []
        for i, window in enumerate(self.layer_windows()):
            prefix = f"model.layers.{i}."
            names = {
                "norm1.weight": prefix + "input_layernorm.weight",
                "norm2.weight": prefix + "post_attention_layernorm.weight",
                "mixer.q": prefix + "self_attn.q_proj.weight",
                "mixer.k": prefix + "self_attn.k_proj.weight",
                "mixer.v": prefix + "self_attn.v_proj.weight",
                "mixer.o": prefix + "self_attn.o_proj.weight",
                "feed_forward.gate": prefix + "mlp.gate_proj.weight",
                "feed_forward.up": prefix + "mlp.up_proj.weight",
                "feed_forward.down": prefix + "mlp.down_proj.weight",
            }
            if self.qk_norm:
                names["mixer.q_norm"] = prefix + "self_attn.q_norm.weight"
                names["mixer.k_norm"] = prefix + "self_attn.k_norm.weight"
            mixer = AttentionSpec(
                hidden_size=self.hidden_size,
                num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim,
                scale=self.head_dim ** -0.5,
                qk_norm=self.qk_norm,
                qk_norm_eps=self.rms_norm_eps,
                position=rope,
                window=window,
            )
            layers.append(prenorm_layer(mixer, ff, norm, norm, names))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            layers=tuple(layers),
            schedule=default_schedule(self.num_hidden_layers),
            final_norm=norm,
            tie_embeddings=self.tie_word_embeddings,
            embed_name="model.embed_tokens.weight",
            final_norm_name="model.norm.weight",
            lm_head_name="lm_head.weight",
            max_position=self.max_position_embeddings,
        )
