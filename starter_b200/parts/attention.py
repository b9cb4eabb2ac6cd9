"""Causal grouped-query attention over the paged cache, with optional per-head q/k norms, rotary
positions and a window.

One step of it: project to q, k, v with one stacked matrix; norm and rotate q and k
per head and file k and v at each token's own position of its sequence; attend from
the cache; project back.  The same code serves a whole prompt, a prompt's later
chunk and a single token, because every query is told its absolute position and
sees exactly the cached keys at or before it (engine/engine.py:665-736, 781-787).
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.layout import KVNeed
from .base import ParamSpec, Part, bytes_of


class GroupedQueryAttention(Part):
    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} key/value heads")
        if spec.head_dim % 2 or spec.head_dim > ops.MAX_HEAD_DIM:
            raise ValueError(f"head_dim {spec.head_dim} must be even and at most {ops.MAX_HEAD_DIM}")
        self.position = position
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.q_norm = self.k_norm = None

    # what this mixer keeps per sequence
    def kv_need(self):
        return KVNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def state_need(self):
        return None

    def param_specs(self):
        s = self.spec
        out = {
            "q": ParamSpec((self.q_size, s.hidden_size)),
            "k": ParamSpec((self.kv_size, s.hidden_size)),
            "v": ParamSpec((self.kv_size, s.hidden_size)),
            "o": ParamSpec((s.hidden_size, self.q_size)),
        }
        if s.qk_norm:
            out["q_norm"] = ParamSpec((s.head_dim,), "gain")
            out["k_norm"] = ParamSpec((s.head_dim,), "gain")
        return out

    def set_params(self, params):
        # one product instead of three; every output is still the same dot product
        # (engine/engine.py:160-162, 171-174)
        self.qkv = torch.cat([params["q"], params["k"], params["v"]], dim=0).contiguous()
        self.o = params["o"].contiguous()
        if self.spec.qk_norm:
            self.q_norm, self.k_norm = params["q_norm"], params["k_norm"]

    def prepare(self, max_position: int) -> bool:
        """Host-side growth before a step; True if device tables were reallocated."""
        if self.position is not None:
            return bool(self.position.ensure(max_position + 1))
        return False

    def _rotation(self):
        if self.position is None:
            return None
        rotation = getattr(self.position, "rotation", None)
        if rotation is None:
            raise ValueError(f"the position part {type(self.position).__name__} offers no rotation(); "
                             "this attention takes rotary positions (or none)")
        return rotation()

    adds_to_stream = True

    def __call__(self, x, ctx, entry, writes_cache=True, add_to=None):
        s = self.spec
        cache = ctx.cache
        keys, values = cache.entry_pages(entry)
        weight = self.qkv if writes_cache else self.qkv[: self.q_size]
        qkv = ops.linear(x, weight, status=ctx.status)
        # the position part says what it turns and how; the kernels take or refuse it by name
        cos, sin = ops.rotation_tables(self._rotation(), s.head_dim)
        if ctx.max_q_len == 1 and ops.decode_from_qkv_takes(s.head_dim, qkv.dtype):
            # one token per sequence: head norm, rotation and cache write inside the attention kernel
            a = ops.attention_decode_qkv(qkv, keys, values, cache.block_table, ctx.seq_slot, ctx.seq_kv_len,
                                         s.num_heads, s.num_kv_heads, s.head_dim, s.scale, s.window,
                                         self.q_norm, self.k_norm, s.qk_norm_eps, cos, sin,
                                         write_cache=writes_cache, kv_hint=ctx.max_kv_len,
                                         # this layer alone writes the pages it reads in this step
                                         early=ctx.fenced and writes_cache)
            return ops.linear(a, self.o, status=ctx.status, add_to=add_to)
        q = ops.qk_norm_rope_store(
            qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.q_norm, self.k_norm, s.qk_norm_eps,
            cos, sin, ctx.tok_pos, ctx.tok_slot, cache.block_table, keys, values,
            write_cache=writes_cache)
        if ctx.max_q_len == 1 and ops.decode_attention_takes(s.head_dim, q.dtype):
            a = ops.attention_decode(q, keys, values, cache.block_table, ctx.seq_slot, ctx.seq_kv_len,
                                     s.num_heads, s.num_kv_heads, s.head_dim, s.scale, s.window,
                                     status=ctx.status, kv_hint=ctx.max_kv_len)
        elif q.dtype == torch.bfloat16 and s.head_dim in ops.PREFILL_HEAD_DIMS:
            a = ops.attention_prefill(q, keys, values, cache.block_table, ctx.seq_slot, ctx.seq_q_start,
                                      ctx.seq_q_len, ctx.seq_kv_len, ctx.tile_seq, ctx.tile_first,
                                      s.num_heads, s.num_kv_heads, s.head_dim, s.scale, s.window,
                                      status=ctx.status, max_q_len=ctx.max_q_len,
                                      blocks=(ctx.block_seq, ctx.block_first))
        else:
            a = ops.attention_rowwise(q, keys, values, cache.block_table, ctx.tok_slot, ctx.tok_pos,
                                      s.num_heads, s.num_kv_heads, s.head_dim, s.scale, s.window)
        return ops.linear(a, self.o, status=ctx.status, add_to=add_to)

    def weight_bytes(self):
        return bytes_of(self.qkv, self.o, self.q_norm, self.k_norm)
