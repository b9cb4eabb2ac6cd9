"""Safetensors reading and writing, the checkpoint check, random model folders (no GPU)."""

import json
import os

import pytest
import torch

from starter_b200.config import config_from_dict
from starter_b200.engine.model import expected_tensors
from starter_b200.weights import (SafetensorsFile, WeightError, load_checkpoint, open_model_files,
                                  place, write_model_folder, write_safetensors)
from tiny import TINY_A, TINY_B, make_folder


def test_safetensors_round_trip_and_agreement_with_the_package(tmp_path):
    from safetensors.torch import load_file, save_file

    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
        "c": torch.arange(6, dtype=torch.int64).view(2, 3), "empty": torch.zeros(0, 4),
    }
    mine = str(tmp_path / "mine.safetensors")
    write_safetensors(mine, tensors, metadata={"k": "v"})
    theirs = load_file(mine)
    for k, v in tensors.items():
        assert torch.equal(theirs[k], v)
    other = str(tmp_path / "theirs.safetensors")
    save_file(tensors, other)
    f = SafetensorsFile(other)
    for k, v in tensors.items():
        assert f.entries[k] == (v.dtype, tuple(v.shape))
        assert torch.equal(f.tensor(k), v)


def test_random_folder_is_a_function_of_seed_and_name(tmp_path):
    a = make_folder(tmp_path / "x", "A", seed=5)
    b = make_folder(tmp_path / "y", "A", seed=5)
    c = make_folder(tmp_path / "z", "A", seed=6)
    fa, fb, fc = (SafetensorsFile(os.path.join(p, "model.safetensors")) for p in (a, b, c))
    assert set(fa.entries) == set(expected_tensors(config_from_dict(TINY_A).to_model_spec()))
    for name in fa.entries:
        assert torch.equal(fa.tensor(name), fb.tensor(name))
    assert not torch.equal(fa.tensor("model.norm.weight"), fc.tensor("model.norm.weight"))
    gains = fa.tensor("model.layers.0.input_layernorm.weight")
    assert abs(gains.mean().item() - 1.0) < 0.1          # 1 + N(0, 0.1)
    assert fa.tensor("model.embed_tokens.weight").std().item() == pytest.approx(0.02, rel=0.1)
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Qwen3ForCausalLM"]
    assert "lm_head.weight" not in fa.entries             # tied
    fb2 = SafetensorsFile(os.path.join(make_folder(tmp_path / "b", "B", seed=1), "model.safetensors"))
    assert fb2.entries["lm_head.weight"][1] == (300, 96)


def _rewrite(folder, change):
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.entries}
    change(tensors)
    del f
    write_safetensors(path, tensors)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(tmp_path, "B", seed=2)

    def spoil(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(16)
        t["model.layers.2.self_attn.k_norm.weight"] = torch.zeros(31)
        t["lm_head.weight"] = torch.zeros(96, 300)

    _rewrite(folder, spoil)
    expected = expected_tensors(config_from_dict(TINY_B).to_model_spec())
    with pytest.raises(WeightError) as info:
        load_checkpoint(folder, expected, torch.float32, "cpu")
    err = info.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert {w[0] for w in err.wrong_shape} == {"model.layers.2.self_attn.k_norm.weight", "lm_head.weight"}
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "[31], expected [32]"):
        assert piece in text


def test_tied_head_may_be_stored_only_if_equal(tmp_path):
    folder = make_folder(tmp_path, "A", seed=3)
    expected = expected_tensors(config_from_dict(TINY_A).to_model_spec())
    alias = ("lm_head.weight", "model.embed_tokens.weight")
    _rewrite(folder, lambda t: t.update({"lm_head.weight": t["model.embed_tokens.weight"].clone()}))
    load_checkpoint(folder, expected, torch.float32, "cpu", tied_alias=alias)
    _rewrite(folder, lambda t: t.update({"lm_head.weight": t["model.embed_tokens.weight"] + 1}))
    with pytest.raises(WeightError, match="ties"):
        load_checkpoint(folder, expected, torch.float32, "cpu", tied_alias=alias)


def test_placement_keeps_bfloat16_int32_and_stored_32_bit_gains():
    m = torch.randn(4, 4)
    assert place(m, "matrix", torch.bfloat16, "cpu").dtype == torch.bfloat16
    assert place(m.to(torch.bfloat16), "matrix", torch.float32, "cpu").dtype == torch.float32
    assert place(torch.ones(4), "gain", torch.bfloat16, "cpu").dtype == torch.float32
    assert place(torch.ones(4).to(torch.bfloat16), "gain", torch.bfloat16, "cpu").dtype == torch.bfloat16
    assert place(torch.arange(4), "matrix", torch.bfloat16, "cpu").dtype == torch.int32


def test_sharded_folder_and_duplicate_names(tmp_path):
    folder = make_folder(tmp_path, "A", seed=4)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    names = list(f.entries)
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fname, group in parts.items():
        write_safetensors(os.path.join(folder, fname), {n: f.tensor(n).clone() for n in group})
    index = {"weight_map": {n: fname for fname, group in parts.items() for n in group}}
    json.dump(index, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    owners = open_model_files(folder)
    assert set(owners) == set(names)
    os.remove(os.path.join(folder, "model.safetensors.index.json"))
    with pytest.raises(ValueError, match="stored in both"):
        open_model_files(folder)


def test_tensor_roles_are_open_and_an_unknown_role_is_an_error():
    import pytest as _pytest
    from starter_b200.parts import ParamSpec, Role, register_role
    from starter_b200.weights.loader import place
    from starter_b200.weights.random_init import random_tensor

    with _pytest.raises(ValueError, match="no tensor role 'decay'"):
        ParamSpec((4,), "decay")
    # a bias is drawn around zero and, stored in 32-bit, stays 32-bit; a matrix follows the working type
    bias = random_tensor(1, "b", ParamSpec((4000,), "bias"), torch.float32)
    assert abs(bias.mean().item()) < 2e-3 and 0.018 < bias.std().item() < 0.022
    assert place(bias, "bias", torch.bfloat16, "cpu").dtype == torch.float32
    assert place(bias, "matrix", torch.bfloat16, "cpu").dtype == torch.bfloat16
    state = random_tensor(1, "s", ParamSpec((4000,), "state"), torch.float32)
    assert 0.09 < state.std().item() < 0.11
    # a part with another kind of tensor registers its role
    register_role("toy_decay", Role(mean=-1.0, std=0.5, keep_32bit=True))
    decay = random_tensor(1, "d", ParamSpec((4000,), "toy_decay"), torch.float32)
    assert -1.05 < decay.mean().item() < -0.95 and 0.45 < decay.std().item() < 0.55


def test_a_layer_spec_must_fit_its_arrangement():
    import pytest as _pytest
    from starter_b200.config import GatedFeedForwardSpec, LayerSpec, ModelSpec, NormSpec, default_schedule
    from starter_b200.config import AttentionSpec, RopeSpec
    from starter_b200.engine.model import expected_tensors

    norm = NormSpec(32, 1e-6)
    attn = AttentionSpec(32, 2, 1, 16, 0.25, False, 1e-6, RopeSpec(16, 1e4))
    ff = GatedFeedForwardSpec(32, 48)
    names = {"mixer.q": "q", "mixer.k": "k", "mixer.v": "v", "mixer.o": "o", "feed_forward.gate": "g",
             "feed_forward.up": "u", "feed_forward.down": "d", "norm1.weight": "n1", "norm2.weight": "n2"}

    def spec_of(layer):
        return ModelSpec("T", 50, 32, (layer,), default_schedule(1), norm, True, "e", "f", "h")

    good = LayerSpec({"mixer": attn, "feed_forward": ff, "norm1": norm, "norm2": norm}, names)
    assert good.mixer is attn and good.norm2 is norm
    assert set(expected_tensors(spec_of(good))) == set(names.values()) | {"e", "f"}
    with _pytest.raises(ValueError, match="lacks \\['norm2'\\]"):
        expected_tensors(spec_of(LayerSpec({"mixer": attn, "feed_forward": ff, "norm1": norm}, names)))
    with _pytest.raises(ValueError, match="has \\['norm9'\\] besides"):
        expected_tensors(spec_of(LayerSpec({"mixer": attn, "feed_forward": ff, "norm1": norm, "norm2": norm,
                                            "norm9": norm}, names)))
    with _pytest.raises(AttributeError, match="no part named 'router'"):
        good.router
