"""Each layer part alone against the plain implementation, and a toy mixer with state of its own,
defined here, registered, built and stepped without touching the library's files."""

from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as plain
from gpu_helpers import DTYPES, assert_close, model_case
from tiny import random_prompt

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def one_sequence_context(runner, n_tokens, slot=None):
    from starter_b200.engine import StepEntry

    slot = runner.open_sequence() if slot is None else slot
    return slot, runner.make_context([StepEntry(slot, [0] * n_tokens, [])])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_parts_of_a_layer_one_by_one(tmp_path_factory, name, dtype):
    from starter_b200.engine import ModelRunner, load_model

    folder, cfg, w32 = model_case(tmp_path_factory, name)
    w = {k: v.to(DT[dtype]) for k, v in w32.items()}
    model = load_model(folder, dtype)
    runner = ModelRunner(model, max_tokens=64 * 8, max_sequences=4)
    layer = cfg["num_hidden_layers"] - 1          # in C this layer has a window
    block = model.blocks[layer]
    prefix = f"model.layers.{layer}."
    tokens = 75
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(tokens, cfg["hidden_size"], generator=gen).to(DT[dtype])
    xd = x.cuda()

    # norm
    want = plain.plain_rms_norm(x, w[prefix + "input_layernorm.weight"], cfg["rms_norm_eps"])
    assert_close(block.norm1(xd), want, dtype, "norm")
    # position tables
    d = plain.head_dim_of(cfg)
    block.mixer.prepare(300)
    cos, sin = plain.plain_rope_tables(cfg["rope_theta"], d, 301, torch.float32)
    assert torch.equal(block.mixer.position.cos[:301].cpu(), cos[:, : d // 2])
    assert torch.equal(block.mixer.position.sin[:301].cpu(), sin[:, : d // 2])
    # feed-forward
    assert_close(block.feed_forward(xd, None), plain.plain_feed_forward(x, w, prefix), dtype, "feed-forward")
    # mixer: a whole sequence in one step, then the same sequence in two steps
    cos_t, sin_t = plain.plain_rope_tables(cfg["rope_theta"], d, tokens, DT[dtype])
    want = plain.plain_mixer(x, w, prefix, cfg, cos_t, sin_t, plain.layer_window(cfg, layer))
    slot, ctx = one_sequence_context(runner, tokens)
    assert_close(block.mixer(xd, ctx, layer, True), want, dtype, "mixer, whole")
    runner.close_sequence(slot)
    slot, ctx = one_sequence_context(runner, 70)
    first = block.mixer(xd[:70].contiguous(), ctx, layer, True)
    _, ctx = one_sequence_context(runner, 5, slot)
    second = block.mixer(xd[70:].contiguous(), ctx, layer, True)
    assert_close(torch.cat([first, second]), want, dtype, "mixer, 70 + 5")
    runner.close_sequence(slot)
    # the whole block
    slot, ctx = one_sequence_context(runner, tokens)
    residual, pending = block(xd.clone(), None, ctx, layer, True)
    cfg_one = dict(cfg)
    want = plain.plain_block(x, w, layer, cfg_one, cos_t, sin_t)
    assert_close((residual.float() + pending.float()), want, dtype, "block")
    runner.close_sequence(slot)


# ----------------------------------------------------------------------------- a toy mixer with state

@dataclass(frozen=True)
class RunningMeanSpec:
    hidden_size: int
    kind: str = "toy_running_mean"


class RunningMeanMixer:
    """y_t = W . mean(x_0 .. x_t): needs no keys, only a running sum and a count per sequence."""

    def __init__(self, spec, dtype, position=None):
        self.spec, self.dtype = spec, dtype

    def param_specs(self):
        from starter_b200.parts import ParamSpec
        return {"w": ParamSpec((self.spec.hidden_size, self.spec.hidden_size))}

    def set_params(self, params):
        self.w = params["w"]

    def kv_need(self):
        return None

    def state_need(self):
        from starter_b200.cache import StateNeed
        return StateNeed((self.spec.hidden_size + 1,), "float32")

    def prepare(self, max_position):
        pass

    def weight_bytes(self):
        return self.w.numel() * self.w.element_size()

    def __call__(self, x, ctx, entry, writes_cache=True):
        state = ctx.cache.entry_state(entry)
        h = self.spec.hidden_size
        if ctx.host is None:
            # a captured step: one token per sequence, nothing of the host may steer it; row i
            # belongs to the sequence in ctx.seq_slot[i]
            slots = ctx.seq_slot.long()
            sums = state[slots, :h] + x.float()
            counts = state[slots, h] + 1
            state[slots, :h] = sums
            state[slots, h] = counts
            return (sums / counts[:, None]).to(x.dtype) @ self.w.t()
        means = torch.empty_like(x, dtype=torch.float32)
        for slot, start, n in zip(ctx.host["seq_slot"].tolist(), ctx.host["seq_q_start"].tolist(),
                                  ctx.host["seq_q_len"].tolist()):
            rows = x[start:start + n].float()
            sums = state[slot, :h] + rows.cumsum(0)
            counts = state[slot, h] + torch.arange(1, n + 1, device=x.device)
            means[start:start + n] = sums / counts[:, None]
            state[slot, :h] = sums[-1]
            state[slot, h] = counts[-1]
        return (means.to(x.dtype) @ self.w.t())


def toy_state_model(dtype, hidden=48, vocab=101):
    """Toy mixer, attention, the toy mixer again (its weights shared, a state of its own), and the
    attention once more reading the keys its first run wrote."""
    from starter_b200.config import (AttentionSpec, GatedFeedForwardSpec, ModelSpec, NormSpec, RopeSpec,
                                     ScheduleEntry, prenorm_layer)
    from starter_b200.engine import DecoderModel
    from starter_b200.parts import register
    from starter_b200.weights import random_checkpoint

    register("mixer", "toy_running_mean", RunningMeanMixer)
    norm = NormSpec(hidden, 1e-5)
    ff = GatedFeedForwardSpec(hidden, 80)
    attn = AttentionSpec(hidden, 3, 1, 16, 0.25, True, 1e-5, RopeSpec(16, 1e4))

    def names(i, mixer_names):
        out = {"norm1.weight": f"l{i}.n1", "norm2.weight": f"l{i}.n2", "feed_forward.gate": f"l{i}.gate",
               "feed_forward.up": f"l{i}.up", "feed_forward.down": f"l{i}.down"}
        out.update({f"mixer.{k}": f"l{i}.{k}" for k in mixer_names})
        return out

    layers = (
        prenorm_layer(RunningMeanSpec(hidden), ff, norm, norm, names(0, ["w"])),
        prenorm_layer(attn, ff, norm, norm, names(1, ["q", "k", "v", "o", "q_norm", "k_norm"])),
    )
    schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 1, writes_cache=False))
    spec = ModelSpec("Toy", vocab, hidden, layers, schedule, norm, True, "embed", "final", "head")
    model = DecoderModel(spec, DT[dtype], "cuda")
    tensors = random_checkpoint(model.expected_tensors(), 3, DT[dtype], "cuda")
    model.load_tensors(tensors)
    return model, tensors, vocab


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_toy_mixer_with_state_registers_builds_and_steps(dtype):
    from starter_b200.engine import ModelRunner, StepEntry

    model, tensors, vocab = toy_state_model(dtype)
    assert model.kv_needs()[0] is None and model.kv_needs()[1] is not None
    runner = ModelRunner(model, max_tokens=64 * 8, max_sequences=4)
    assert set(runner.cache.state) == {0, 2} and len(runner.cache.groups) == 1

    a, b = random_prompt(70, vocab, 1), random_prompt(9, vocab, 2)
    sa, sb = runner.open_sequence(), runner.open_sequence()
    whole = runner.step([StepEntry(sa, a, list(range(70))), StepEntry(sb, b, list(range(9)))])
    runner.close_sequence(sa)
    runner.close_sequence(sb)
    # the same two requests cut differently, in slots that were just used: state must start at zero
    sb, sa = runner.open_sequence(), runner.open_sequence()
    rows_a = [runner.step([StepEntry(sa, a[:66], list(range(66)))])]
    rows_b = []
    for i in range(4):
        out = runner.step([StepEntry(sa, [a[66 + i]], [0]), StepEntry(sb, b[2 * i:2 * i + 2], [0, 1])])
        rows_a.append(out[:1])
        rows_b.append(out[1:])
    rows_b.append(runner.step([StepEntry(sb, b[8:], [0])]))
    assert_close(torch.cat(rows_a + rows_b), whole, dtype, "toy model, cut in steps")
    # and the toy layer does what it says: compare its first run with plain torch
    x = model.embed[torch.tensor(b, device="cuda")].float()
    n1 = plain.plain_rms_norm(x.to(DT[dtype]).cpu(), tensors["l0.n1"].cpu(), 1e-5).float()
    means = n1.cumsum(0) / torch.arange(1, 10)[:, None]
    want = means.to(DT[dtype]) @ tensors["l0.w"].cpu().t()
    s = runner.open_sequence()
    ctx = runner.make_context([StepEntry(s, b, [])])
    got = model.blocks[0].mixer(model.blocks[0].norm1(model.embed[torch.tensor(b, device="cuda")].contiguous()), ctx, 0, True)
    assert_close(got, want, dtype, "toy mixer alone")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_toy_mixer_with_state_runs_in_the_captured_step(dtype):
    """Generation (captured, self-feeding steps) with a mixer that keeps a running state: the graphs
    are captured in the middle of generation, whenever the batch reaches a new length class, and the
    warm-up runs of a capture must leave the state as they found it.  Tokens and the logits of every
    step equal the eager run's."""
    from starter_b200.engine.entry import Engine
    from starter_b200.engine.generate import Request

    model, _, vocab = toy_state_model(dtype)
    prompts = [random_prompt(60, vocab, 11), random_prompt(20, vocab, 12), random_prompt(1, vocab, 13)]
    new = 80      # every sequence crosses a page edge; the batch passes the classes of 1, 2 and 3 pages

    def run(engine):
        requests = [Request(list(p), new) for p in prompts]
        loop = engine._ensure_room(requests, len(requests))
        loop.lookahead = False        # each step's logits are read before the next step runs
        tokens, rows = [], []
        for n, step_out in enumerate(loop.stream_batch(requests)):
            tokens.append([step_out[i] for i in range(len(prompts))])
            graphs = engine.runner.graphs
            if n > 0 and graphs is not None:
                rows.append(graphs.logits[graphs.last_key].clone())
        return tokens, rows

    engine = Engine.from_model(model, max_batch=4)
    captured, rows = run(engine)
    assert len(engine.runner.graphs.graphs) >= 3
    engine.runner.check_status()
    # the eager run of the same loop, fed the captured run's tokens, step by step
    from starter_b200.engine import StepEntry
    runner = engine.runner
    slots = [runner.open_sequence() for _ in prompts]
    first = runner.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    assert first.argmax(-1).tolist() == captured[0]
    for n, got in enumerate(rows):
        eager = runner.step([StepEntry(s, [captured[n][i]], [0]) for i, s in enumerate(slots)])
        assert_close(got, eager, dtype, f"captured against eager, step {n + 1}")
        if dtype == "float32":
            assert eager.argmax(-1).tolist() == captured[n + 1]
    for s in slots:
        runner.close_sequence(s)
    again, _ = run(engine)                   # slots and states used again: nothing carried over
    assert again == captured


# ----------------------------------------------------------------------------- an arrangement of its own

class SandwichBlock:
    """A block with a third norm, on the mixer's output before it joins the residual stream:
    ``x1 = x + norm3(mixer(norm1(x)))``, ``x2 = x1 + feed_forward(norm2(x1))``."""

    FAMILIES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm",
                "norm3": "norm"}

    def __init__(self, parts):
        self._parts = dict(parts)
        self.mixer = parts["mixer"]

    def parts(self):
        return dict(self._parts)

    def __call__(self, residual, pending, ctx, entry, writes_cache=True):
        p = self._parts
        n = p["norm1"].add(residual, pending)
        a = p["norm3"](p["mixer"](n, ctx, entry, writes_cache))
        m = p["norm2"].add(residual, a)
        return residual, p["feed_forward"](m, ctx)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_layer_with_three_norms_builds_from_its_spec(dtype):
    from starter_b200.config import (AttentionSpec, GatedFeedForwardSpec, LayerSpec, ModelSpec, NormSpec,
                                     RopeSpec, default_schedule)
    from starter_b200.engine import DecoderModel, ModelRunner, StepEntry
    from starter_b200.parts import register
    from starter_b200.weights import random_checkpoint

    register("arrangement", "toy_sandwich", SandwichBlock)
    hidden, vocab = 64, 131
    norm = NormSpec(hidden, 1e-6)
    attn = AttentionSpec(hidden, 4, 2, 16, 0.25, True, 1e-6, RopeSpec(16, 1e4))
    ff = GatedFeedForwardSpec(hidden, 96)
    names = {f"mixer.{k}": f"a.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
    names.update({f"feed_forward.{k}": f"f.{k}" for k in ("gate", "up", "down")})
    names.update({f"norm{i}.weight": f"n{i}" for i in (1, 2, 3)})
    layer = LayerSpec({"mixer": attn, "feed_forward": ff, "norm1": norm, "norm2": norm, "norm3": norm},
                      names, arrangement="toy_sandwich")
    spec = ModelSpec("Toy3", vocab, hidden, (layer,), default_schedule(1), norm, True, "embed", "final", "head")
    model = DecoderModel(spec, DT[dtype], "cuda")
    assert "n3" in model.expected_tensors()
    tensors = random_checkpoint(model.expected_tensors(), 9, DT[dtype], "cuda")
    model.load_tensors(tensors)
    runner = ModelRunner(model, max_tokens=64 * 4, max_sequences=2)
    seq = random_prompt(80, vocab, 4)
    s = runner.open_sequence()
    whole = runner.step([StepEntry(s, seq, list(range(80)))])
    runner.close_sequence(s)
    s = runner.open_sequence()
    parts = [runner.step([StepEntry(s, seq[:50], list(range(50)))])]
    parts += [runner.step([StepEntry(s, [t], [0])]) for t in seq[50:]]
    assert_close(torch.cat(parts), whole, dtype, "sandwich layer, cut in steps")
    # against plain torch: the plain block with the third norm put in
    w = {k: v.cpu() for k, v in tensors.items()}
    renamed = {f"L.self_attn.{k}_proj.weight": w[f"a.{k}"] for k in "qkvo"}
    renamed.update({f"L.self_attn.{k}_norm.weight": w[f"a.{k}_norm"] for k in "qk"})
    renamed.update({f"L.mlp.{k}_proj.weight": w[f"f.{k}"] for k in ("gate", "up", "down")})
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, hidden_size=hidden)
    x = w["embed"][torch.tensor(seq)]
    cos, sin = plain.plain_rope_tables(1e4, 16, len(seq), x.dtype)
    a = plain.plain_mixer(plain.plain_rms_norm(x, w["n1"], 1e-6), renamed, "L.", cfg, cos, sin, None)
    x = x + plain.plain_rms_norm(a, w["n3"], 1e-6)
    x = x + plain.plain_feed_forward(plain.plain_rms_norm(x, w["n2"], 1e-6), renamed, "L.")
    want = torch.nn.functional.linear(plain.plain_rms_norm(x, w["final"], 1e-6), w["embed"]).float()
    assert_close(whole, want, dtype, "sandwich layer against plain torch")
    # a layer spec that does not fit its arrangement is refused by name
    bad = LayerSpec({"mixer": attn, "feed_forward": ff, "norm1": norm, "norm2": norm}, names, "toy_sandwich")
    with pytest.raises(ValueError, match="norm3"):
        DecoderModel(ModelSpec("T", vocab, hidden, (bad,), default_schedule(1), norm, True, "e", "f", "h"),
                     DT[dtype], "cuda")


def test_a_rotation_the_kernels_cannot_do_is_refused_by_name():
    from starter_b200 import ops
    from starter_b200.parts import Rotation

    cos = torch.ones(8, 4, device="cuda")
    assert ops.rotation_tables(None, 16) == (None, None)
    assert ops.rotation_tables(Rotation(cos, cos, 8), 8)[0] is cos
    with pytest.raises(ops.KernelError, match="half-split"):
        ops.rotation_tables(Rotation(cos, cos, 8, "interleaved"), 8)
    with pytest.raises(ops.KernelError, match="whole head"):
        ops.rotation_tables(Rotation(cos, cos, 8), 16)


# ----------------------------------------------------------------------------- more toy parts

@dataclass(frozen=True)
class RoutedFeedForwardSpec:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    kind: str = "toy_routed"


class RoutedFeedForward:
    """Top-1 routing over small gated experts; router logits and the choice in float32."""

    def __init__(self, spec, dtype):
        self.spec, self.dtype = spec, dtype

    def param_specs(self):
        from starter_b200.parts import ParamSpec
        s = self.spec
        out = {"router": ParamSpec((s.num_experts, s.hidden_size))}
        for e in range(s.num_experts):
            out[f"gate_up{e}"] = ParamSpec((2 * s.intermediate_size, s.hidden_size))
            out[f"down{e}"] = ParamSpec((s.hidden_size, s.intermediate_size))
        return out

    def set_params(self, params):
        self.p = params

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.p.values())

    def __call__(self, x, ctx=None):
        from starter_b200 import ops
        choice = (x.float() @ self.p["router"].float().t()).argmax(-1)
        out = torch.zeros_like(x)
        for e in range(self.spec.num_experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                xe = x[rows].contiguous()
                out[rows] = ops.linear(ops.linear(xe, self.p[f"gate_up{e}"], gated=True), self.p[f"down{e}"])
        return out


@dataclass(frozen=True)
class ScaledRopeSpec:
    head_dim: int
    theta: float
    factor: float
    kind: str = "toy_scaled_rope"


def scaled_rope_class():
    from starter_b200.parts import RotaryTable

    class ScaledRope(RotaryTable):
        """Rotary positions with every position divided by a factor (position interpolation)."""

        def ensure(self, length):
            if length <= self.length:
                return False
            size = max(64, self.length)
            while size < length:
                size *= 2
            freqs = self.angles(self.spec.theta, self.spec.head_dim, size) / self.spec.factor
            self.cos = freqs.cos().contiguous().to(self.device)
            self.sin = freqs.sin().contiguous().to(self.device)
            self.length = size
            return True

    return ScaledRope


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_routed_feed_forward_and_another_position_encoding_plug_in(dtype):
    """A model whose layers differ: attention with scaled rotary positions + routed experts, then the
    library's attention with its own rotary positions + the dense feed-forward.  Built from specs,
    stepped whole and in pieces, and the first layer checked against plain torch."""
    from starter_b200.config import (AttentionSpec, GatedFeedForwardSpec, ModelSpec, NormSpec,
                                     RopeSpec, default_schedule, prenorm_layer)
    from starter_b200.engine import DecoderModel, ModelRunner, StepEntry
    from starter_b200.parts import register
    from starter_b200.weights import random_checkpoint

    register("feed_forward", "toy_routed", RoutedFeedForward)
    register("position", "toy_scaled_rope", scaled_rope_class())
    hidden, vocab = 64, 97
    norm = NormSpec(hidden, 1e-6)

    def attn(position):
        return AttentionSpec(hidden, 4, 2, 16, 0.25, True, 1e-6, position)

    def names(i, ff_names):
        out = {"norm1.weight": f"l{i}.n1", "norm2.weight": f"l{i}.n2"}
        out.update({f"mixer.{k}": f"l{i}.attn.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")})
        out.update({f"feed_forward.{k}": f"l{i}.ff.{k}" for k in ff_names})
        return out

    routed = RoutedFeedForwardSpec(hidden, 48, 3)
    routed_names = ["router"] + [f"{k}{e}" for e in range(3) for k in ("gate_up", "down")]
    layers = (
        prenorm_layer(attn(ScaledRopeSpec(16, 1e4, 4.0)), routed, norm, norm, names(0, routed_names)),
        prenorm_layer(attn(RopeSpec(16, 1e4)), GatedFeedForwardSpec(hidden, 80), norm, norm, names(1, ["gate", "up", "down"])),
    )
    spec = ModelSpec("Toy2", vocab, hidden, layers, default_schedule(2), norm, False, "embed", "final", "head")
    model = DecoderModel(spec, DT[dtype], "cuda")
    tensors = random_checkpoint(model.expected_tensors(), 5, DT[dtype], "cuda")
    model.load_tensors(tensors)
    assert len(model.positions) == 2                     # two position parts, not shared
    runner = ModelRunner(model, max_tokens=64 * 4, max_sequences=4)
    seq = random_prompt(90, vocab, 3)
    s = runner.open_sequence()
    whole = runner.step([StepEntry(s, seq, list(range(90)))])
    runner.close_sequence(s)
    s = runner.open_sequence()
    parts = [runner.step([StepEntry(s, seq[:70], list(range(70)))])]
    parts += [runner.step([StepEntry(s, [t], [0])]) for t in seq[70:]]
    assert_close(torch.cat(parts), whole, dtype, "toy model 2, cut in steps")
    # the scaled positions really are used: the first layer's mixer equals the plain mixer run with
    # tables of positions / 4
    w = {k: v.cpu() for k, v in tensors.items()}
    x = torch.randn(12, hidden, generator=torch.Generator().manual_seed(1)).to(DT[dtype])
    cos, sin = plain.plain_rope_tables(1e4, 16, 12, torch.float32)
    freqs = torch.outer(torch.arange(12).float(), 1.0 / (1e4 ** (torch.arange(0, 16, 2).float() / 16))) / 4.0
    emb = torch.cat((freqs, freqs), -1)
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, hidden_size=hidden)
    renamed = {f"model.layers.0.self_attn.{k}_proj.weight": w[f"l0.attn.{k}"] for k in "qkvo"}
    renamed.update({f"model.layers.0.self_attn.{k}_norm.weight": w[f"l0.attn.{k}_norm"] for k in "qk"})
    want = plain.plain_mixer(x, renamed, "model.layers.0.", cfg, emb.cos().to(DT[dtype]), emb.sin().to(DT[dtype]), None)
    slot, ctx = one_sequence_context(runner, 12)
    got = model.blocks[0].mixer(x.cuda(), ctx, 0, True)
    assert_close(got, want, dtype, "mixer with scaled rotary positions")
