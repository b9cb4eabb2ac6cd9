"""The generic decoder: an embedding, layers built from parts, a run order, a final norm and a head.

Everything model-specific arrives in the ``ModelSpec``.  ``expected_tensors``
derives from the spec the checkpoint names and shapes the model wants; ``forward``
runs one step over a packed batch (see ``starter_b200.engine.batch``) and returns
float32 logits for the wanted rows only, as the reference computes the head for
the last position only (engine/engine.py:801-803).
"""

from __future__ import annotations

import torch

from .. import ops
from ..parts import ParamSpec, lookup


def build_layers(spec, dtype, device):
    """Instantiate every layer's parts; position parts with equal specs are shared.

    The layer's arrangement names the parts it is made of and their families; each part's spec is
    looked up under that family by its ``kind``.  A part whose spec carries a ``position`` spec is
    handed the position part built from it."""
    positions = {}
    blocks = []
    for index, layer in enumerate(spec.layers):
        arrangement = lookup("arrangement", layer.arrangement)
        wanted = dict(arrangement.FAMILIES)
        missing = [n for n in wanted if n not in layer.parts]
        extra = [n for n in layer.parts if n not in wanted]
        if missing or extra:
            raise ValueError(f"layer {index}: the {layer.arrangement!r} arrangement is made of "
                             f"{sorted(wanted)}; the layer spec lacks {missing} and has {extra} besides")
        built = {}
        for name, family in wanted.items():
            part_spec = layer.parts[name]
            cls = lookup(family, part_spec.kind)
            pos_spec = getattr(part_spec, "position", None)
            if pos_spec is not None and pos_spec not in positions:
                positions[pos_spec] = lookup("position", pos_spec.kind)(pos_spec, dtype, device)
            if family == "mixer":
                built[name] = cls(part_spec, dtype, positions.get(pos_spec))
            else:
                built[name] = cls(part_spec, dtype)
        blocks.append(arrangement(built))
    return blocks, list(positions.values())


def _layer_params(block, names: dict) -> dict:
    """``{checkpoint name: (part name, logical name, ParamSpec)}`` for one block."""
    out = {}
    for part_name, part in block.parts().items():
        for logical, pspec in part.param_specs().items():
            key = f"{part_name}.{logical}"
            if key not in names:
                raise ValueError(f"the layer spec names no checkpoint tensor for {key}")
            out[names[key]] = (part_name, logical, pspec)
    return out


def expected_tensors(spec) -> dict:
    """``{checkpoint name: ParamSpec}`` in a fixed order: embedding, layers, final norm, head."""
    blocks, _ = build_layers(spec, torch.float32, "cpu")
    out = {spec.embed_name: ParamSpec((spec.vocab_size, spec.hidden_size))}
    for block, layer in zip(blocks, spec.layers):
        for name, (_, _, pspec) in _layer_params(block, layer.names).items():
            out[name] = pspec
    out[spec.final_norm_name] = ParamSpec((spec.final_norm.size,), "gain")
    if not spec.tie_embeddings:
        out[spec.lm_head_name] = ParamSpec((spec.vocab_size, spec.hidden_size))
    return out


class DecoderModel:
    def __init__(self, spec, dtype, device="cuda"):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks, self.positions = build_layers(spec, dtype, self.device)
        self.final_norm = lookup("norm", spec.final_norm.kind)(spec.final_norm, dtype)
        self.embed = None
        self.lm_head = None
        for entry in spec.schedule:
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"the run order names layer {entry.layer}; the model has {len(self.blocks)}")
        writers = {}
        for entry in spec.schedule:
            if entry.writes_cache:
                writers.setdefault(entry.cache, entry.layer)
        for entry in spec.schedule:
            if not entry.writes_cache and entry.cache not in writers:
                raise ValueError(f"cache entry {entry.cache} is read but no entry of the run order writes it")

    # ------------------------------------------------------------------ weights

    def expected_tensors(self) -> dict:
        return expected_tensors(self.spec)

    def load_tensors(self, tensors) -> None:
        """Take a mapping ``checkpoint name -> device tensor`` (a dict, or the loader's mapping that
        places a tensor when it is asked for).  Layers are taken one at a time and a layer's tensors
        are let go of as soon as its parts have them (stacked where a part stacks), so loading never
        holds two copies of more than one layer."""
        spec = self.spec
        self.embed = tensors[spec.embed_name]
        self.lm_head = self.embed if spec.tie_embeddings else tensors[spec.lm_head_name]
        self.final_norm.set_params({"weight": tensors[spec.final_norm_name]})
        for block, layer in zip(self.blocks, spec.layers):
            grouped = {}
            wanted = _layer_params(block, layer.names)
            for name, (part_name, logical, _) in wanted.items():
                grouped.setdefault(part_name, {})[logical] = tensors[name]
            for part_name, part in block.parts().items():
                if part.param_specs():
                    part.set_params(grouped[part_name])
            del grouped
            for name in wanted:
                tensors.pop(name, None)

    # ------------------------------------------------------------------ cache needs

    def kv_needs(self) -> dict:
        """``{cache entry: KVNeed}``, taken from the entry's writer."""
        needs = {}
        for entry in self.spec.schedule:
            if entry.writes_cache and entry.cache not in needs:
                needs[entry.cache] = self.blocks[entry.layer].mixer.kv_need()
        return needs

    def state_needs(self) -> dict:
        needs = {}
        for entry in self.spec.schedule:
            if entry.writes_cache and entry.cache not in needs:
                needs[entry.cache] = self.blocks[entry.layer].mixer.state_need()
        return needs

    # ------------------------------------------------------------------ compute

    def prepare(self, max_position: int) -> bool:
        """Host-side growth (position tables) that must not happen in the middle of a step.  True if
        any device table moved: graphs captured before then hold stale addresses."""
        moved = False
        for block in self.blocks:
            for part in block.parts().values():
                prepare = getattr(part, "prepare", None)
                if prepare is not None:
                    moved = bool(prepare(max_position)) or moved
        return moved

    def hidden(self, ctx):
        """Run the layers; returns ``(residual, pending)`` with the last sum still open."""
        # the step's first kernel is an ordinary launch: the fence behind which the step's other
        # kernels may read early what earlier steps left (lengths, cache pages)
        residual = ops.embedding(ctx.tokens, self.embed, ctx.status, fence=True)
        ctx.fenced = True
        pending = None
        for entry in self.spec.schedule:
            residual, pending = self.blocks[entry.layer](residual, pending, ctx, entry.cache,
                                                         entry.writes_cache)
        return residual, pending

    def logits(self, residual, pending, rows, status=None):
        """Float32 logits ``[len(rows), vocab]`` of the rows asked for."""
        h = self.final_norm.add_rows(residual, pending, rows)
        return ops.linear(h, self.lm_head, out_float=True, status=status)

    def forward(self, ctx, rows):
        residual, pending = self.hidden(ctx)
        if rows is None or rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        return self.logits(residual, pending, rows, ctx.status)

    def step_weight_bytes(self) -> int:
        """Bytes of weights one decode step reads: every layer the run order names, each time it is
        named, the final norm and the head (the embedding table is only gathered from)."""
        total = self.final_norm.weight_bytes() + self.lm_head.numel() * self.lm_head.element_size()
        for entry in self.spec.schedule:
            total += sum(p.weight_bytes() for p in self.blocks[entry.layer].parts().values())
        return total
