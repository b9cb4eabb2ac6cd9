"""Python face of the CUDA kernels: argument checks, output allocation, launch on the current stream.

Every function here runs a hand-written kernel from ``starter_b200/csrc`` (the one
exception: a bfloat16 matrix product of 129 to 511 rows goes to the vendor's GEMM
library, where the reference uses one too, engine/engine.py:431-450).  There is no
CPU path: tensors must live on a CUDA device, and a shape a kernel cannot take is
refused with an error that names it.
"""

from __future__ import annotations

import ctypes
import functools

import torch

from .cache.layout import PAGE_TOKENS
from .csrc import build

SMALL_ROWS = 16
#: Up to this many rows the bfloat16 product runs on this library's few-row tcgen05 kernel
#: (csrc/gemm_tcgen05.cu), where it is bound by streaming the weights.  Measured on the four
#: projections of a 2560-wide layer: 63-70 us a layer up to 64 rows against 64-86 for the vendor's
#: library; 66 against 68-77 at 96 rows, 70 against 68 at 128, 95-102 against 73 at 192.
TENSOR_CORE_MAX_ROWS = 128
#: From this many rows on it runs on this library's persistent CTA-pair kernel
#: (csrc/gemm_prompt_tcgen05.cu), whose tiles are 256 rows high.  Measured a layer against the
#: vendor's library (which needs a separate SwiGLU kernel): 114 against 106 us at 512 rows, 167
#: against 164 at 1,024, 298 against 307 at 2,048, 434 against 470 at 3,072; at 256 rows 100 against
#: 75.  In between (129 to 511 rows) the vendor's GEMM is used, as the reference does from 33 rows on
#: (engine/engine.py:431-450).
PROMPT_MIN_ROWS = 512
MAX_HEAD_DIM = 256

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


_checked = set()


def _lib(name: str):
    """The kernel library of ``name.cu``; refuses one compiled for another cache page size."""
    lib = build.load(name)
    if name not in _checked:
        compiled = lib.sb_page_tokens()
        if compiled != PAGE_TOKENS:
            raise KernelError(f"libsb_{name} was compiled for cache pages of {compiled} tokens, the cache "
                              f"uses pages of {PAGE_TOKENS}")
        _checked.add(name)
    return lib


def _code(dtype) -> int:
    if dtype not in _DT:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")
    return _DT[dtype]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


try:                                   # the raw handle of the current stream without building objects
    _raw_stream = torch._C._cuda_getCurrentRawStream
    _current_device = torch._C._cuda_getDevice
except AttributeError:                 # pragma: no cover - older or newer torch: the public way
    _raw_stream = _current_device = None


def _stream():
    """The current CUDA stream as a ``void*`` (called once per launch: it has to be cheap)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(_current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, name, dtype=None, ndim=None):
    # the common case first and in one expression: this runs several times per launch
    try:
        if (t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype)
                and (ndim is None or t.dim() == ndim)):
            return
    except AttributeError:
        pass
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU implementation)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")


class _Added:
    """What ``linear`` returns when it has put its result onto ``add_to`` instead of returning it."""

    def __repr__(self):
        return "ADDED"


#: the value that stands for "already added onto the residual stream" (see ``linear``'s ``add_to``)
ADDED = _Added()

#: how many kernels of this library have been launched by this process (library GEMMs not counted)
launch_count = 0
#: switch for the decode attention's reads before its dependent-launch wait (see attention_decode_qkv)
EARLY_READS = True


def _check(rc, what, kernels=1):
    global launch_count
    launch_count += kernels
    if rc != 0:
        if rc == -1:
            raise KernelError(f"{what}: this combination of dtypes has no kernel")
        if rc == -2:
            raise KernelError(f"{what}: a size is outside what the kernel takes")
        raise KernelError(f"{what}: launch failed with CUDA error {rc}")


def _gain_code(x, gain):
    if gain.dtype == torch.float32:
        return 0
    if gain.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"a {gain.dtype} gain cannot scale {x.dtype} activations")


# ---------------------------------------------------------------------------------------- rows

def embedding(tokens, table, status=None, fence=False):
    """``out[t] = table[tokens[t]]``; ``tokens`` int32 ``[T]``, ``table`` ``[V, H]``.

    ``fence``: launch it as an ordinary kernel (not a dependent launch), so that it starts only when
    everything before it on the stream has completed.  As a step's first kernel it is what lets later
    kernels of the step read, before their own dependent-launch wait, what earlier steps wrote."""
    _need(tokens, "tokens", torch.int32, 1)
    _need(table, "table", None, 2)
    out = torch.empty((tokens.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
    rc = _lib("elementwise").sb_embedding(
        _code(table.dtype), _ptr(tokens), _ptr(table), _ptr(out), tokens.shape[0], table.shape[1],
        table.shape[0], _ptr(status), int(fence), _stream())
    _check(rc, "embedding")
    return out


def rmsnorm(x, gain, eps, delta=None, rows=None, out=None):
    """RMSNorm of the rows of ``x`` ``[T, H]``.

    With ``delta`` the norm is taken of ``x + delta`` and, unless ``rows`` is given,
    ``x`` is replaced by that sum (the residual stream).  With ``rows`` (int32
    ``[R]``) only those rows are normed and ``x`` is left alone.
    """
    _need(x, "x", None, 2)
    _need(gain, "gain", None, 1)
    hidden = x.shape[1]
    if gain.shape[0] != hidden:
        raise KernelError(f"gain has {gain.shape[0]} entries for rows of {hidden}")
    if delta is not None:
        _need(delta, "delta", x.dtype, 2)
        if delta.shape != x.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match x {tuple(x.shape)}")
    n_rows = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.shape[0]
    if out is None:
        out = torch.empty((n_rows, hidden), dtype=x.dtype, device=x.device)
    rc = _lib("elementwise").sb_rmsnorm(
        _code(x.dtype), _gain_code(x, gain), _ptr(x), _ptr(delta), _ptr(gain), _ptr(out), _ptr(rows),
        n_rows, hidden, ctypes.c_float(eps), _stream())
    _check(rc, "rmsnorm")
    return out


def swiglu(gate_up):
    """``round(silu(gate)) * up`` for ``gate_up = [gate | up]`` of shape ``[T, 2 * I]``."""
    _need(gate_up, "gate_up", None, 2)
    if gate_up.shape[1] % 2:
        raise KernelError(f"gate_up has an odd width {gate_up.shape[1]}")
    inner = gate_up.shape[1] // 2
    out = torch.empty((gate_up.shape[0], inner), dtype=gate_up.dtype, device=gate_up.device)
    rc = _lib("elementwise").sb_swiglu(
        _code(gate_up.dtype), _ptr(gate_up), _ptr(out), gate_up.shape[0], inner, _stream())
    _check(rc, "swiglu")
    return out


# ---------------------------------------------------------------------------------------- matrix products

def linear(x, weight, out_float=False, gated=False, status=None, add_to=None):
    """``x @ weight.T`` for ``x`` ``[T, K]`` and ``weight`` ``[N, K]`` (no bias).

    ``add_to`` (``[T, N]``, the residual stream) is an offer, not an order: where the kernel that
    runs has an epilogue for it (the prompt product), ``add_to`` becomes
    ``round(add_to + round(product))`` in place and ``ADDED`` is returned; otherwise ``add_to`` is
    left alone and the product is returned as usual.

    ``gated``: ``weight`` is ``[gate; up]`` stacked (``[2 * I, K]``) and the result is
    ``round(silu(x @ gate.T)) * (x @ up.T)`` of shape ``[T, I]``.  ``out_float``
    returns float32 whatever the working type (used for logits).  ``status`` (int32 ``[1]``) is the
    device word in which the tensor-core kernel reports a wait that ran out.
    """
    _need(x, "x", None, 2)
    _need(weight, "weight", x.dtype, 2)
    rows, k_dim = x.shape
    if weight.shape[1] != k_dim:
        raise KernelError(f"weight {tuple(weight.shape)} does not take inputs of width {k_dim}")
    n_total = weight.shape[0]
    if gated and n_total % 2:
        raise KernelError(f"a gated weight needs an even number of rows, got {n_total}")
    n_out = n_total // 2 if gated else n_total
    dt = _code(x.dtype)
    if dt == 1 and rows <= TENSOR_CORE_MAX_ROWS and tensor_core_ok(x, weight, gated, n_out):
        return linear_tensor_core(x, weight, out_float=out_float, gated=gated, status=status)
    if rows <= SMALL_ROWS:
        out_dtype = torch.float32 if (out_float or dt == 0) else x.dtype
        if gated and out_float and dt == 1:
            raise KernelError("a gated product cannot return float32 from bfloat16")
        y = torch.empty((rows, n_out), dtype=out_dtype, device=x.device)
        rc = _lib("linear_small").sb_linear_small(
            dt, int(out_float), int(gated), _ptr(x), _ptr(weight), _ptr(y), rows, n_out, k_dim,
            _stream())
        _check(rc, "linear_small")
        return y
    if dt == 0:
        y = torch.empty((rows, n_total), dtype=torch.float32, device=x.device)
        rc = _lib("sgemm").sb_sgemm_nt(_ptr(x), _ptr(weight), _ptr(y), rows, n_total, k_dim,
                                             _stream())
        _check(rc, "sgemm")
    elif out_float:
        y = torch.mm(x, weight.t(), out_dtype=torch.float32)
    elif rows >= PROMPT_MIN_ROWS and k_dim % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        if (add_to is not None and not gated and add_to.dtype == torch.bfloat16 and add_to.is_contiguous()
                and tuple(add_to.shape) == (rows, n_out)):
            linear_prompt(x, weight, status=status, residual=add_to)
            return ADDED
        return linear_prompt(x, weight, gated=gated, status=status)
    else:
        y = torch.mm(x, weight.t())
    return swiglu(y) if gated else y


def tensor_core_ok(x, weight, gated, n_out) -> bool:
    """Whether the tcgen05 product takes these operands: k a multiple of 8 (16-byte rows for TMA),
    16-byte aligned bases, gated widths in steps of 64."""
    k_dim = x.shape[1]
    if k_dim % 8 or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return False
    if gated and n_out % 64:
        return False
    return True


@functools.lru_cache(maxsize=4096)     # asked once per launch, with the same few shapes step after step
def gemm_plan(rows: int, n_out: int, k_dim: int, gated: bool):
    """``(bm, splits, stages)``: activation rows per tile; how many CTAs (one cluster) share a tile's
    k range; how deep the ring of shared-memory stages is.

    With few rows the product is bound by streaming the weights: about two CTAs per SM should be
    loading, each with some 100 KB in flight.  With more rows two or three CTAs per SM hold 128-row tiles."""
    bm = 16
    while bm < rows and bm < 128:
        bm *= 2
    tiles = (n_out // 64 if gated else -(-n_out // 128)) * -(-rows // bm)
    k_blocks = -(-k_dim // 64)
    stage_bytes = 16384 + bm * 128
    if rows <= 64:
        def fits(splits, stages):       # every CTA resident at once
            return tiles * splits <= 148 * ((227 * 1024) // (stages * stage_bytes + 2048))

        # Measured inside the captured decode step (not kernel by kernel: what a product can have on
        # its way before its predecessor ends depends on the room that predecessor leaves on an SM).
        if tiles * 6 <= 148 and k_blocks >= 32:
            # few tiles (a narrow output): eight CTAs a tile with six stages, two to an SM; where
            # the stages are too large for that, six CTAs a tile with the deepest ring
            return (bm, 8, 6) if fits(8, 6) else (bm, min(6, 148 // tiles), 8)
        if tiles <= 74 and k_blocks >= 32:
            # up to half as many tiles as SMs: six stages, two CTAs to an SM, about 1.3 CTAs per SM
            splits = max(1, min(8, k_blocks // 4, 192 // tiles))
            if fits(splits, 6):
                return bm, splits, 6
        # otherwise: rings deeper than four stages lose (fewer CTAs fit on an SM); the product is
        # fastest with about 80% of the CTA slots taken and all CTAs resident at once; when three
        # stages let a third CTA onto each SM and that buys clearly more CTAs, three stages win
        def choice(stages):
            slots = 148 * ((227 * 1024) // (stages * stage_bytes + 2048))
            return slots, max(1, min(8, k_blocks // 4, int(0.82 * slots) // tiles))

        slots4, splits4 = choice(4)
        slots3, splits3 = choice(3)
        if bm > 16 and slots3 > slots4 and (tiles > slots4 or tiles * splits3 > 1.5 * tiles * splits4):
            stages, splits = 3, splits3
        else:
            stages, splits = 4, splits4
    else:
        # measured at 96 to 500 rows (128-row tiles).  Few tiles: one CTA of six stages per SM and up
        # to four CTAs sharing a tile's k range.  More tiles than SMs: two stages (three CTAs on an
        # SM), and two CTAs a tile while there is one row tile.  In between: three stages.
        slots3 = 148 * ((227 * 1024) // (3 * stage_bytes + 2048))
        if tiles <= 74:
            # (clusters of three were measured far slower than of two or four here)
            splits = max(1, min(4, k_blocks // 8, 148 // tiles))
            stages, splits = 6, (2 if splits == 3 else splits)
        elif tiles > 148:
            stages, splits = 2, (2 if rows <= 128 and k_blocks >= 16 else 1)
        else:
            stages, splits = 3, max(1, min(4, k_blocks // 8, slots3 // tiles))
    return bm, splits, stages


def linear_tensor_core(x, weight, out_float=False, gated=False, bm=None, splits=None, stages=None,
                       status=None, withhold=None):
    """The bfloat16 product on tcgen05 tensor cores (csrc/gemm_tcgen05.cu).

    ``withhold = (k_block, limit_ns)`` is for tests of the kernel's give-up path: the activation copy
    of that k-block is left out, so a wait inside the kernel runs out after ``limit_ns``; the kernel
    returns, bit 4 of ``status`` is set and the result is undefined."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    rows, k_dim = x.shape
    n_total = weight.shape[0]
    n_out = n_total // 2 if gated else n_total
    if weight.shape[1] != k_dim:
        raise KernelError(f"weight {tuple(weight.shape)} does not take inputs of width {k_dim}")
    if not tensor_core_ok(x, weight, gated, n_out):
        raise KernelError(f"the tensor-core product needs k % 8 == 0, 16-byte aligned operands and gated "
                          f"widths in steps of 64; got k = {k_dim}, n = {n_out}")
    plan = gemm_plan(rows, n_out, k_dim, gated)
    bm = bm or plan[0]
    splits = splits or plan[1]
    stages = stages or max(plan[2], -(-bm * 512 // (16384 + bm * 128)))
    stages = min(stages, (226 * 1024) // (16384 + bm * 128))     # a tile height other than the plan's
    out = torch.empty((rows, n_out), dtype=torch.float32 if out_float else torch.bfloat16, device=x.device)
    if withhold is not None:
        rc = _lib("gemm_tcgen05").sb_gemm_tcgen05_withheld(
            _ptr(x), _ptr(weight), _ptr(out), rows, n_out, k_dim, bm, splits, stages, int(gated),
            int(out_float), _ptr(status), ctypes.c_ulonglong(int(withhold[1])), int(withhold[0]), _stream())
    else:
        rc = _lib("gemm_tcgen05").sb_gemm_tcgen05(
            _ptr(x), _ptr(weight), _ptr(out), rows, n_out, k_dim, bm, splits, stages, int(gated),
            int(out_float), _ptr(status), _stream())
    if rc in (-3, -4):
        raise KernelError("the TMA descriptors for the tensor-core product could not be made "
                          f"(code {rc}); is the driver too old for cuTensorMapEncodeTiled?")
    _check(rc, "gemm_tcgen05")
    return out


def linear_prompt(x, weight, gated=False, bn=0, pairs=0, status=None, withhold=None, residual=None):
    """The bfloat16 product for many rows: the persistent CTA-pair kernel (csrc/gemm_prompt_tcgen05.cu).

    ``bn`` is the number of weight rows per tile (0: chosen by the kernel's host side), ``pairs`` the
    number of CTA pairs (0: one per two SMs).  ``withhold = (k_block, limit_ns)`` is for tests of the
    give-up path: one weight copy is left out, a wait runs out after ``limit_ns``, the kernel returns,
    bit 4 of ``status`` is set and the result is undefined.  With ``residual`` (``[rows, n]``
    bfloat16, not with ``gated``) the result is ``round(residual + round(product))``, written into
    ``residual`` itself, which is returned."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    rows, k_dim = x.shape
    n_total = weight.shape[0]
    n_out = n_total // 2 if gated else n_total
    if weight.shape[1] != k_dim:
        raise KernelError(f"weight {tuple(weight.shape)} does not take inputs of width {k_dim}")
    if k_dim % 8 or (gated and n_total % 2) or x.data_ptr() % 16 or weight.data_ptr() % 16:
        raise KernelError(f"the prompt product needs k % 8 == 0 and 16-byte aligned operands; got k = {k_dim}")
    if residual is not None:
        _need(residual, "residual", torch.bfloat16, 2)
        if gated or tuple(residual.shape) != (rows, n_out) or withhold is not None:
            raise KernelError(f"a residual of shape {tuple(residual.shape)} cannot take a "
                              f"{'gated ' if gated else ''}product of shape {(rows, n_out)}")
        out = residual
    else:
        out = torch.empty((rows, n_out), dtype=torch.bfloat16, device=x.device)
    lib = _lib("gemm_prompt_tcgen05")
    if withhold is not None:
        rc = lib.sb_gemm_prompt_withheld(_ptr(x), _ptr(weight), _ptr(out), rows, n_out, k_dim, int(bn), int(pairs),
                                         int(gated), _ptr(status), ctypes.c_ulonglong(int(withhold[1])),
                                         int(withhold[0]), _stream())
    else:
        rc = lib.sb_gemm_prompt(_ptr(x), _ptr(weight), _ptr(out), _ptr(residual), rows, n_out, k_dim, int(bn), int(pairs),
                                int(gated), _ptr(status), _stream())
    if rc in (-3, -4):
        raise KernelError("the TMA descriptors for the prompt product could not be made "
                          f"(code {rc}); is the driver too old for cuTensorMapEncodeTiled?")
    _check(rc, "gemm_prompt_tcgen05")
    return out


# ---------------------------------------------------------------------------------------- attention

def rotation_tables(rotation, head_dim: int):
    """``(cos, sin)`` for the kernels from a position part's ``Rotation`` (or ``(None, None)``).

    The kernels here (``qk_norm_rope_store`` and the decode attention that rotates the new token
    itself) turn the whole head in half-split layout; anything else is refused by name."""
    if rotation is None:
        return None, None
    if rotation.layout != "half_split" or rotation.rotary_dim != head_dim:
        raise KernelError(f"the kernels rotate the whole head ({head_dim} dimensions) in half-split layout; "
                          f"asked for {rotation.rotary_dim} dimensions in {rotation.layout!r} layout")
    return rotation.cos, rotation.sin


def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_gain, k_gain, eps, cos_table, sin_table,
                       tok_pos, tok_slot, block_table, k_store, v_store, write_cache=True):
    """Norm and rotate the query and key heads of ``qkv`` and file keys and values in the cache.

    ``qkv`` is ``[T, (heads + 2 * kv_heads) * head_dim]`` (queries alone,
    ``[T, heads * head_dim]``, when ``write_cache`` is false); returns the queries
    ``[T, heads * head_dim]``.  ``k_store``/``v_store`` are one cache entry's pages
    ``[pages, kv_heads, 64, head_dim]``; ``block_table`` int32 ``[slots, max_pages]``.
    """
    _need(qkv, "qkv", None, 2)
    n_tokens = qkv.shape[0]
    width = (heads + 2 * kv_heads) * head_dim if write_cache else heads * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"qkv has width {qkv.shape[1]}, expected {width}")
    if head_dim % 2 or head_dim > MAX_HEAD_DIM:
        raise KernelError(f"head_dim {head_dim} must be even and at most {MAX_HEAD_DIM}")
    _need(tok_pos, "tok_pos", torch.int32, 1)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    gain_code = 0
    for g in (q_gain, k_gain):
        if g is not None:
            _need(g, "head gain", None, 1)
            if g.shape[0] != head_dim:
                raise KernelError(f"head gain has {g.shape[0]} entries for head_dim {head_dim}")
            gain_code = _gain_code(qkv, g)
    if (q_gain is None) != (k_gain is None):
        raise KernelError("q and k head norms come together")
    if cos_table is not None:
        _need(cos_table, "cos_table", torch.float32, 2)
        _need(sin_table, "sin_table", torch.float32, 2)
        if cos_table.shape[1] != head_dim // 2 or sin_table.shape != cos_table.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
    if write_cache:
        for store in (k_store, v_store):
            _need(store, "cache pages", qkv.dtype, 4)
            if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
                raise KernelError(f"cache pages have shape {tuple(store.shape)}, expected "
                                  f"[pages, {kv_heads}, {PAGE_TOKENS}, {head_dim}]")
    q_out = torch.empty((n_tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    rc = _lib("rope_cache").sb_qk_norm_rope_store(
        _code(qkv.dtype), gain_code, _ptr(qkv), _ptr(q_out), _ptr(q_gain), _ptr(k_gain),
        _ptr(cos_table), _ptr(sin_table), _ptr(tok_pos), _ptr(tok_slot), _ptr(block_table),
        block_table.shape[1], _ptr(k_store if write_cache else None),
        _ptr(v_store if write_cache else None), n_tokens, heads, kv_heads, head_dim,
        ctypes.c_float(eps), int(write_cache), qkv.shape[1], _stream())
    _check(rc, "qk_norm_rope_store")
    return q_out


def attention_rowwise(q, k_store, v_store, block_table, tok_slot, tok_pos, heads, kv_heads, head_dim,
                      scale, window=None):
    """Causal attention of each query row over its sequence's cached keys (plain kernel)."""
    _need(q, "q", None, 2)
    if q.shape[1] != heads * head_dim:
        raise KernelError(f"q has width {q.shape[1]}, expected {heads * head_dim}")
    if head_dim > MAX_HEAD_DIM:
        raise KernelError(f"head_dim {head_dim} exceeds {MAX_HEAD_DIM}")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    for store in (k_store, v_store):
        _need(store, "cache pages", q.dtype, 4)
        if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    out = torch.empty_like(q)
    rc = _lib("attention_rowwise").sb_attention_rowwise(
        _code(q.dtype), _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
        block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), q.shape[0], heads, kv_heads, head_dim,
        ctypes.c_float(scale), int(window or 0), _stream())
    _check(rc, "attention_rowwise")
    return out


PREFILL_HEAD_DIMS = (16, 32, 64, 128)


def attention_prefill(q, k_store, v_store, block_table, seq_slot, seq_q_start, seq_q_len, seq_kv_len,
                      tile_seq, tile_first, heads, kv_heads, head_dim, scale, window=None, status=None,
                      kernel=None, max_q_len=None, blocks=None, withhold=None):
    """Causal attention for steps with many tokens per sequence (bfloat16, tensor cores).

    ``q`` ``[T, heads * head_dim]`` packed by sequence; the ``seq_*`` arrays describe each sequence
    of the step, ``tile_seq``/``tile_first`` list the tiles of 64 queries.  Head sizes 64 and 128 run
    on the tcgen05 kernel (256 queries a block, S and O in tensor memory) when some sequence brings
    more than 128 queries (``max_q_len``, taken as large when not given); everything else runs on
    the mma.sync kernel, which has the smaller blocks.  ``kernel`` ("tcgen05" or "mma") forces one.
    ``blocks = (block_seq, block_first)`` is the same work list in blocks of 256 queries, which is what
    the tcgen05 kernel launches; without it that kernel is launched once per tile of 64 and three of
    four launches find nothing to do.  ``withhold = (step, limit_ns)`` is for tests of the tcgen05
    kernel's give-up path: half of the values of that step of 128 keys are not copied, the wait on them
    runs out after ``limit_ns``, bit 16 of ``status`` is set and the result is undefined."""
    _need(q, "q", torch.bfloat16, 2)
    if q.shape[1] != heads * head_dim:
        raise KernelError(f"q has width {q.shape[1]}, expected {heads * head_dim}")
    if head_dim not in PREFILL_HEAD_DIMS:
        raise KernelError(f"head_dim {head_dim} is not one of {PREFILL_HEAD_DIMS}")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    for store in (k_store, v_store):
        _need(store, "cache pages", q.dtype, 4)
        if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for name, t in (("seq_slot", seq_slot), ("seq_q_start", seq_q_start), ("seq_q_len", seq_q_len),
                    ("seq_kv_len", seq_kv_len), ("tile_seq", tile_seq), ("tile_first", tile_first)):
        _need(t, name, torch.int32, 1)
    out = torch.empty_like(q)
    if kernel is None:
        long_enough = max_q_len is None or max_q_len > 128
        kernel = "tcgen05" if head_dim in PREFILL_TC_HEAD_DIMS and long_enough else "mma"
    if kernel == "tcgen05":
        if head_dim not in PREFILL_TC_HEAD_DIMS:
            raise KernelError(f"the tcgen05 prefill kernel takes head_dim {PREFILL_TC_HEAD_DIMS}, not {head_dim}")
        if not q.is_contiguous():
            raise KernelError("q must be contiguous")
        own_list = blocks is not None and blocks[0] is not None
        if own_list:
            for name, t in (("block_seq", blocks[0]), ("block_first", blocks[1])):
                _need(t, name, torch.int32, 1)
        list_seq, list_first = blocks if own_list else (tile_seq, tile_first)
        if withhold is not None:
            _lib("attention_prefill_tc").sb_attention_prefill_tc_withhold(
                int(withhold[0]), ctypes.c_ulonglong(int(withhold[1])))
        rc = _lib("attention_prefill_tc").sb_attention_prefill_tc(
            _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table), block_table.shape[1],
            _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(list_seq),
            _ptr(list_first), list_seq.shape[0], q.shape[0], k_store.shape[0], heads, kv_heads, head_dim,
            ctypes.c_float(scale), int(window or 0), _ptr(status) if status is not None else None,
            int(own_list), _stream())
        _check(rc, "attention_prefill_tc")
        return out
    rc = _lib("attention_prefill").sb_attention_prefill(
        _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table), block_table.shape[1],
        _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(tile_seq),
        _ptr(tile_first), tile_seq.shape[0], heads, kv_heads, head_dim, ctypes.c_float(scale),
        int(window or 0), _stream())
    _check(rc, "attention_prefill")
    return out


PREFILL_TC_HEAD_DIMS = (64, 128)
DECODE_CLUSTER_SPLITS = 8
DECODE_HEAD_DIMS = (16, 32, 64, 128, 256)


def decode_attention_takes(head_dim: int, dtype) -> bool:
    """Whether the split-key decode kernel takes this head size: 16 elements per lane, and two
    stages of a page's keys and values (2 * 2 * 64 * head_dim elements) within shared memory."""
    return head_dim in DECODE_HEAD_DIMS and head_dim * dtype.itemsize <= 512


@functools.lru_cache(maxsize=4096)
def decode_splits(rows: int, kv_heads: int, groups: int, group_rows: int = 4, kv_hint: int = 0) -> int:
    """How many parts to cut each row's keys into, so that every block is resident at once and the
    SMs are busy.

    The tensor-core kernel (``group_rows`` 16) merges up to ``DECODE_CLUSTER_SPLITS`` parts inside a
    thread-block cluster at no extra launch, and every part may be as short as a page.  Measured
    inside the captured decode step at 3,073 keys: the step is fastest with at most 256 blocks (two
    fit on an SM, 296 in all, but 280 or 288 blocks cost 12-17% of the whole step at 5, 6 and 12
    rows), with 224 rather than 256 when that means 7 parts instead of 8, and with no more than 8
    parts at 3,073 keys: 17 parts through scratch memory and the merge kernel lose 1-2% of the step
    to 8 in a cluster at 1 and 2 rows.  The CUDA-core kernel always merges with a second kernel and
    wants three pages per part."""
    blocks = rows * kv_heads * (-(-groups // group_rows))
    pages = -(-kv_hint // PAGE_TOKENS) if kv_hint > 0 else None
    if group_rows < 16:
        want = max(1, min(32, (2 * 148) // blocks))
        return want if pages is None else max(1, min(want, -(-pages // 3)))
    want = max(1, min(DECODE_CLUSTER_SPLITS, 256 // blocks))
    if want > 4 and want * blocks > 240:
        want -= 1
    if pages is None:
        return want
    want = max(1, min(want, pages))
    # Few rows of many keys: 8 parts a row leave most SMs without a block, and a block streams about
    # 60 GB/s.  More parts through scratch memory cost a merge kernel (3 us) and fill the SMs.
    # Estimated both ways in microseconds from the bytes (a page of keys and values of a 128-wide
    # head is 32 KB) and taken when the estimate says so; the crossover it gives for one row of 8
    # key/value heads, 6,700 keys, lies between the measured 3,073 (cluster faster by 0.7 us a
    # layer) and 16,384 (scratch faster by 6.2 us).
    more = max(1, min(32, 256 // blocks, pages // 3))
    if more >= 12 and more > want:
        megabytes = blocks * pages * 0.032768
        in_cluster = megabytes / min(6.5, want * blocks * 0.06)
        through_scratch = 3.0 + megabytes / min(6.5, more * blocks * 0.06)
        if through_scratch < in_cluster:
            return more
    return want


def decode_from_qkv_takes(head_dim: int, dtype) -> bool:
    """Whether ``attention_decode_qkv`` takes this head size and type (the tensor-core decode kernel)."""
    return dtype == torch.bfloat16 and head_dim in PREFILL_HEAD_DIMS


def attention_decode_qkv(qkv, k_store, v_store, block_table, row_slot, row_kv_len, heads, kv_heads, head_dim,
                         scale, window, q_gain, k_gain, eps, cos_table, sin_table, write_cache=True,
                         n_splits=None, kv_hint=0, early=False):
    """One-token attention straight from the q/k/v product (bfloat16, tensor cores): head norm,
    rotation and the cache write of ``qk_norm_rope_store`` happen inside the attention kernel, with
    the same arithmetic.  Row ``i`` of ``qkv`` is the new token of the sequence in ``row_slot[i]``, at
    position ``row_kv_len[i] - 1``.  ``qkv`` holds the queries alone when ``write_cache`` is false.

    ``early``: the caller vouches that ``row_kv_len``, the page table and every cached key and value
    but the new token's were complete before this step's first kernel started (``embedding(...,
    fence=True)``) and that nothing else in this step writes them; the kernel then reads the lengths
    and the page numbers before its dependent-launch wait, while the q/k/v product still runs."""
    _need(qkv, "qkv", torch.bfloat16, 2)
    if not decode_from_qkv_takes(head_dim, qkv.dtype):
        raise KernelError(f"head_dim {head_dim} is not one of {PREFILL_HEAD_DIMS}")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    rows = qkv.shape[0]
    width = (heads + 2 * kv_heads) * head_dim if write_cache else heads * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"qkv has width {qkv.shape[1]}, expected {width}")
    for store in (k_store, v_store):
        _need(store, "cache pages", qkv.dtype, 4)
        if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(row_slot, "row_slot", torch.int32, 1)
    _need(row_kv_len, "row_kv_len", torch.int32, 1)
    gain_code = 0
    if (q_gain is None) != (k_gain is None):
        raise KernelError("q and k head norms come together")
    for g in (q_gain, k_gain):
        if g is not None:
            _need(g, "head gain", None, 1)
            if g.shape[0] != head_dim:
                raise KernelError(f"head gain has {g.shape[0]} entries for head_dim {head_dim}")
            gain_code = _gain_code(qkv, g)
    if cos_table is not None:
        _need(cos_table, "cos_table", torch.float32, 2)
        _need(sin_table, "sin_table", torch.float32, 2)
        if cos_table.shape[1] != head_dim // 2 or sin_table.shape != cos_table.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
    if n_splits is None:
        n_splits = decode_splits(rows, kv_heads, heads // kv_heads, 16, kv_hint)
    out = torch.empty((rows, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    part_acc = part_ml = None
    in_cluster = 1 < n_splits <= DECODE_CLUSTER_SPLITS
    if n_splits > 1 and not in_cluster:
        part_acc = torch.empty((rows * heads * n_splits * head_dim,), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((rows * heads * n_splits * 2,), dtype=torch.float32, device=qkv.device)
    rc = _lib("attention_decode_mma").sb_attention_decode_mma_fused(
        _ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
        block_table.shape[1], _ptr(row_slot), _ptr(row_kv_len), rows, heads, kv_heads, head_dim,
        ctypes.c_float(scale), int(window or 0), n_splits, _ptr(part_acc), _ptr(part_ml), _ptr(q_gain),
        _ptr(k_gain), gain_code, ctypes.c_float(eps), _ptr(cos_table), _ptr(sin_table), int(write_cache),
        int(bool(early) and write_cache and EARLY_READS), _stream())
    _check(rc, "attention_decode_fused", 2 if n_splits > 1 and not in_cluster else 1)
    return out


def attention_decode(q, k_store, v_store, block_table, row_slot, row_kv_len, heads, kv_heads, head_dim,
                     scale, window=None, n_splits=None, status=None, kv_hint=0, withhold=None):
    """One query per row (the newest token of its sequence) over that sequence's cached keys.

    ``row_kv_len[r]`` is the sequence's length with the query's own key already filed; the lengths
    stay on the device.  ``head_dim`` must be one of ``DECODE_HEAD_DIMS``.

    ``withhold = (page, limit_ns)`` is for tests of the CUDA-core kernel's give-up path: the values of
    that page of every block's range are not copied, the wait on them runs out after ``limit_ns``,
    the kernel returns with bit 8 of ``status`` set and the result is undefined."""
    _need(q, "q", None, 2)
    rows = q.shape[0]
    if q.shape[1] != heads * head_dim:
        raise KernelError(f"q has width {q.shape[1]}, expected {heads * head_dim}")
    if not decode_attention_takes(head_dim, q.dtype):
        raise KernelError(f"head_dim {head_dim} in {q.dtype} is outside what the decode kernel takes: "
                          f"one of {DECODE_HEAD_DIMS} and at most 512 bytes per head row")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    for store in (k_store, v_store):
        _need(store, "cache pages", q.dtype, 4)
        if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(row_slot, "row_slot", torch.int32, 1)
    _need(row_kv_len, "row_kv_len", torch.int32, 1)
    tensor_cores = q.dtype == torch.bfloat16 and head_dim in PREFILL_HEAD_DIMS
    if n_splits is None:
        n_splits = decode_splits(rows, kv_heads, heads // kv_heads, 16 if tensor_cores else 4, kv_hint)
    out = torch.empty_like(q)
    part_acc = part_ml = None
    # up to DECODE_CLUSTER_SPLITS splits of the tensor-core kernel are one thread-block cluster and
    # merge through distributed shared memory; more go through scratch and a merge kernel
    in_cluster = tensor_cores and 1 < n_splits <= DECODE_CLUSTER_SPLITS
    if n_splits > 1 and not in_cluster:
        part_acc = torch.empty((rows * heads * n_splits * head_dim,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((rows * heads * n_splits * 2,), dtype=torch.float32, device=q.device)
    if tensor_cores:
        rc = _lib("attention_decode_mma").sb_attention_decode_mma(
            _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table), block_table.shape[1],
            _ptr(row_slot), _ptr(row_kv_len), rows, heads, kv_heads, head_dim, ctypes.c_float(scale),
            int(window or 0), n_splits, _ptr(part_acc), _ptr(part_ml), _stream())
    else:
        if withhold is not None:
            _lib("attention_decode").sb_attention_decode_withhold(int(withhold[0]), ctypes.c_ulonglong(int(withhold[1])))
        rc = _lib("attention_decode").sb_attention_decode(
            _code(q.dtype), _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
            block_table.shape[1], _ptr(row_slot), _ptr(row_kv_len), rows, heads, kv_heads, head_dim,
            ctypes.c_float(scale), int(window or 0), n_splits, _ptr(part_acc), _ptr(part_ml),
            _ptr(status), _stream())
    _check(rc, "attention_decode", 2 if n_splits > 1 and not in_cluster else 1)
    return out


# ---------------------------------------------------------------------------------------- sampling

def sample(logits, temperature=None, request_key=None, position=None, status=None, out=None, feed=None):
    """One token per row of float32 ``logits`` ``[B, V]``: argmax, or a draw where temperature > 0.

    ``feed = (tokens, positions, lengths)`` (int32 ``[B]`` each): the drawn token is also stored as
    the row's next input and its position and length are advanced by one."""
    _need(logits, "logits", torch.float32, 2)
    rows, vocab = logits.shape
    if temperature is not None:
        _need(temperature, "temperature", torch.float32, 1)
        _need(request_key, "request_key", torch.int32, 1)
        _need(position, "position", torch.int32, 1)
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    chunks = lib.sb_sample_chunks(vocab)
    cand_v = torch.empty((rows * chunks,), dtype=torch.float32, device=logits.device)
    cand_i = torch.empty((rows * chunks,), dtype=torch.int32, device=logits.device)
    rc = lib.sb_sample(
        _ptr(logits), rows, vocab, ctypes.c_longlong(logits.stride(0)), _ptr(temperature),
        _ptr(request_key), _ptr(position), _ptr(out), _ptr(status),
        _ptr(feed[0] if feed else None), _ptr(feed[1] if feed else None),
        _ptr(feed[2] if feed else None), _ptr(cand_v), _ptr(cand_i), _stream())
    _check(rc, "sample", 2)
    return out


# ---------------------------------------------------------------------------------------- chains

CHAIN_MAX_ROWS = 64
CHAIN_MAX_STAGES = 8
CHAIN_MAX_LINEAR = 6
CHAIN_STATUS_BIT = 32
_chain_state = {}      # device index -> {"sync": int64[2], "partial": float32 arena}


def _chain_scratch(device, floats: int):
    """The chains of one device share two 64-bit words (grid-barrier counter, give-up flag) and one
    float arena for partial tiles.  A chain writes the arena only after the kernel before it on the
    stream has completed, so consecutive chains can use the same memory."""
    state = _chain_state.get(device.index)
    if state is None:
        state = _chain_state[device.index] = {
            "sync": torch.zeros((2,), dtype=torch.int64, device=device), "partial": None}
    if state["partial"] is None or state["partial"].numel() < floats:
        state["partial"] = torch.empty((max(floats, 1 << 20),), dtype=torch.float32, device=device)
    return state["sync"], state["partial"]


def reset_chains(device=None) -> None:
    """Clear the chains' shared words after a chain gave up (its barrier count is then off and every
    later chain on the device gives up at once until this is called)."""
    for index, state in _chain_state.items():
        if device is None or torch.device(device).index in (None, index):
            state["sync"].zero_()


class ChainValue:
    """A ``[rows, width]`` bfloat16 tensor that a chain which is still open will produce.  ``resolve``
    launches the chain and gives the tensor."""

    __slots__ = ("chain", "stage", "tensor", "shape")

    def __init__(self, chain, stage, tensor, shape):
        self.chain, self.stage, self.tensor, self.shape = chain, stage, tensor, shape

    @property
    def dtype(self):
        return torch.bfloat16


def resolve(value):
    """The tensor behind ``value``: a tensor as it is, a ``ChainValue`` after its chain has run."""
    if isinstance(value, ChainValue):
        value.chain.close()
        if value.tensor is None:
            raise KernelError("this value was summed straight into the norm after it and was never stored")
        return value.tensor
    return value


def chain_takes_linear(x, weight, gated: bool) -> bool:
    """Whether a chain can run ``x @ weight.T``: bfloat16, at most 64 rows, 16-byte aligned operands,
    k a multiple of 8, a gated width a multiple of 64."""
    rows, k_dim = x.shape
    n_total = weight.shape[0]
    if weight.dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or not 1 <= rows <= CHAIN_MAX_ROWS:
        return False
    if k_dim % 8 or weight.data_ptr() % 16 or not weight.is_contiguous() or weight.shape[1] != k_dim:
        return False
    if gated and (n_total % 2 or (n_total // 2) % 64):
        return False
    return True


def chain_takes_norm(hidden: int, gain) -> bool:
    return hidden % 8 == 0 and hidden <= 16384 and gain.dtype in (torch.float32, torch.bfloat16) \
        and gain.data_ptr() % 16 == 0


class OpenChain:
    """Few-row projections and row norms that run as ONE persistent kernel (csrc/dense_chain.cu).

    Stages are added with ``linear`` and ``add_norm`` and run when the chain is closed (by ``close`` or
    by ``resolve`` of one of its values).  A stage may read tensors that exist when the chain is
    launched and values of earlier stages of the same chain."""

    def __init__(self, rows: int, device, status=None):
        if not 1 <= rows <= CHAIN_MAX_ROWS:
            raise KernelError(f"a chain runs 1 to {CHAIN_MAX_ROWS} rows, not {rows}")
        self.rows, self.device, self.status = rows, device, status
        self.stages = []
        self.closed = False
        #: None, or a zeroed int64 tensor [ctas, 64]: each CTA's time stamps (ns) at its stage boundaries
        self.trace = None
        self.n_ctas = _lib("dense_chain").sb_dense_chain_ctas()
        self.bm = 16 if rows <= 16 else 32 if rows <= 32 else 64

    # ------------------------------------------------------------------ building

    def room_for(self, linear: bool) -> bool:
        if self.closed or len(self.stages) >= CHAIN_MAX_STAGES:
            return False
        return not linear or sum(s["kind"] == 0 for s in self.stages) < CHAIN_MAX_LINEAR

    def _input(self, x, what):
        """(tensor, keep-alive) of a stage input: a tensor, or a stored value of this chain."""
        if isinstance(x, ChainValue):
            if x.chain is not self:
                return resolve(x)
            if x.tensor is None:
                raise KernelError(f"{what} was summed straight into a norm and cannot be read again")
            return x.tensor
        return x

    def linear(self, x, weight, gated=False) -> ChainValue:
        shape = x.shape
        xt = self._input(x, "the input of a projection")
        _need(xt, "x", torch.bfloat16, 2)
        _need(weight, "weight", torch.bfloat16, 2)
        if not chain_takes_linear(xt, weight, gated) or shape[0] != self.rows or not self.room_for(True):
            raise KernelError("this projection does not fit the chain (see chain_takes_linear)")
        n_out = weight.shape[0] // 2 if gated else weight.shape[0]
        out = torch.empty((self.rows, n_out), dtype=torch.bfloat16, device=self.device)
        parts = _lib("dense_chain").sb_dense_chain_parts(n_out, x.shape[1], int(gated), self.n_ctas)
        tiles = n_out // 64 if gated else -(-n_out // 128)
        self.stages.append({"kind": 0, "n_out": n_out, "k_dim": x.shape[1], "gated": int(gated), "store": 1,
                            "x": xt, "w": weight, "out": out, "parts": parts,
                            "floats": tiles * parts * self.bm * 128})
        return ChainValue(self, len(self.stages) - 1, out, (self.rows, n_out))

    def add_norm(self, residual, delta, gain, eps) -> ChainValue:
        """``residual += delta`` (in place, rounded) and its RMSNorm; ``delta`` None norms ``residual``
        alone; ``residual`` None norms ``delta`` alone.  A ``delta`` that is the value of the stage just
        before, a plain projection, is summed from that stage's partial tiles and never stored."""
        hidden = (residual if residual is not None else delta).shape[1]
        if not chain_takes_norm(hidden, gain) or not self.room_for(False):
            raise KernelError("this norm does not fit the chain (see chain_takes_norm)")
        fused = (isinstance(delta, ChainValue) and delta.chain is self and delta.stage == len(self.stages) - 1
                 and self.stages[-1]["kind"] == 0 and not self.stages[-1]["gated"] and delta.tensor is not None)
        if fused:
            self.stages[-1]["store"] = 0
            self.stages[-1]["out"] = None
            delta.tensor = None
            dt = None
        else:
            dt = self._input(delta, "the delta of a norm") if delta is not None else None
        if residual is not None:
            _need(residual, "residual", torch.bfloat16, 2)
        if dt is not None:
            _need(dt, "delta", torch.bfloat16, 2)
        normed = torch.empty((self.rows, hidden), dtype=torch.bfloat16, device=self.device)
        self.stages.append({"kind": 1, "hidden": hidden, "gain": gain, "eps": float(eps), "residual": residual,
                            "delta": dt, "normed": normed})
        return ChainValue(self, len(self.stages) - 1, normed, (self.rows, hidden))

    # ------------------------------------------------------------------ running

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        if not self.stages:
            return
        floats = sum(s.get("floats", 0) for s in self.stages)
        sync, arena = _chain_scratch(self.device, floats)
        desc = (ctypes.c_longlong * (16 * len(self.stages)))()
        eps = (ctypes.c_float * len(self.stages))()
        at = 0
        for i, s in enumerate(self.stages):
            d = [0] * 16
            if s["kind"] == 0:
                partial = arena.data_ptr() + 4 * at
                at += s["floats"]
                d[:10] = [0, s["n_out"], s["k_dim"], s["gated"], s["store"], s["x"].data_ptr(), s["w"].data_ptr(),
                          s["out"].data_ptr() if s["out"] is not None else 0, partial, s["parts"]]
            else:
                d[:8] = [1, s["hidden"], int(s["gain"].dtype == torch.float32), int(s["residual"] is not None),
                         s["residual"].data_ptr() if s["residual"] is not None else 0,
                         s["delta"].data_ptr() if s["delta"] is not None else 0, s["gain"].data_ptr(),
                         s["normed"].data_ptr()]
                eps[i] = s["eps"]
            for j, v in enumerate(d):
                desc[16 * i + j] = v
        rc = _lib("dense_chain").sb_dense_chain(
            desc, eps, len(self.stages), self.rows, _ptr(sync), _ptr(self.status), ctypes.c_ulonglong(0),
            _ptr(self.trace), _stream())
        if rc in (-3, -4):
            raise KernelError(f"the TMA descriptors for a chain could not be made (code {rc})")
        _check(rc, "dense_chain")
