"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory at the point where they need attention
(all memory handed to another allocator, a serving loop that must not take the allocator's lock, a
plugin without allocation rights), so ``sb_attention_decode_noalloc`` keeps its split-key scratch in
a fixed array inside the library.  This file is collected last on purpose: it is one small addition
and must not stand in the way of the other tests.
"""

import contextlib
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = dict(atol=2e-2, rtol=2e-2)


@contextlib.contextmanager
def _nothing_else_frees():
    """Device memory is compared before and after a call; meanwhile nothing else may give memory back
    (the collector freeing an earlier test's CUDA graph would), so collect first and hold it off."""
    gc.collect()
    torch.cuda.synchronize()
    gc.disable()
    try:
        yield
    finally:
        gc.enable()


def _case(seed, lengths, heads, kv_heads, d):
    """Random paged keys/values and one query per sequence; returns device tensors."""
    gen = torch.Generator().manual_seed(seed)
    n_pages = sum((n + 63) // 64 for n in lengths) + 2
    perm = torch.randperm(n_pages, generator=gen).tolist()
    ks = torch.randn(n_pages, kv_heads, 64, d, generator=gen).to(torch.bfloat16)
    vs = torch.randn(n_pages, kv_heads, 64, d, generator=gen).to(torch.bfloat16)
    table = torch.zeros(len(lengths), 8, dtype=torch.int32)
    at = 0
    for s, n in enumerate(lengths):
        for p in range((n + 63) // 64):
            table[s, p] = perm[at]
            at += 1
    q = torch.randn(len(lengths), heads * d, generator=gen).to(torch.bfloat16)
    dev = lambda t: t.cuda()
    return dict(q=dev(q), ks=dev(ks), vs=dev(vs), table=dev(table),
                slot=dev(torch.arange(len(lengths), dtype=torch.int32)),
                kv_len=dev(torch.tensor(lengths, dtype=torch.int32)))


def _call(lib, c, heads, kv_heads, d, splits, out=None):
    out = torch.empty_like(c["q"]) if out is None else out
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.sb_attention_decode_noalloc(
        ptr(c["q"]), ptr(out), ptr(c["ks"]), ptr(c["vs"]), ptr(c["table"]), c["table"].shape[1],
        ptr(c["slot"]), ptr(c["kv_len"]), c["q"].shape[0], heads, kv_heads, d, ctypes.c_float(d ** -0.5),
        0, splits, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row():
    from starter_b200 import ops
    from starter_b200.csrc import build

    lib = build.load("attention_decode_noalloc")
    lib.sb_attention_decode_noalloc_message.restype = ctypes.c_char_p
    heads, kv_heads, d = 8, 2, 64
    # two calls in a row with different inputs and different numbers of splits: the second must not
    # be disturbed by what the first left in the shared array
    for seed, lengths, splits in ((1, [200, 1, 64, 130], 5), (2, [65, 300], 3)):
        c = _case(seed, lengths, heads, kv_heads, d)
        want = ops.attention_decode(c["q"], c["ks"], c["vs"], c["table"], c["slot"], c["kv_len"], heads,
                                    kv_heads, d, d ** -0.5, None, splits)
        got = torch.empty_like(c["q"])
        # the first launch of a kernel loads its code, which may take device memory; the call that
        # is held to "device memory does not move" is therefore the second of the same kind
        _call(lib, c, heads, kv_heads, d, splits, out=torch.empty_like(c["q"]))
        with _nothing_else_frees():
            free_before = torch.cuda.mem_get_info()[0]
            rc, got = _call(lib, c, heads, kv_heads, d, splits, out=got)
            torch.cuda.synchronize()
            free_after = torch.cuda.mem_get_info()[0]
        assert rc == 0, lib.sb_attention_decode_noalloc_message()
        assert free_after == free_before
        assert torch.allclose(got.float(), want.float(), **TOL)
    # calls that do go through the shared array (more than 8 parts are merged by a second kernel that
    # reads them from it): two in a row, of different shapes, so that the second call's entries lie
    # over the first call's at other offsets; several parts of the short sequences see no key at all
    for seed, lengths, h, kvh, dim, splits in ((4, [500, 70, 1, 333], 8, 2, 64, 12),
                                               (5, [129, 512, 64], 6, 3, 128, 20),
                                               (6, [500, 70, 1, 333], 8, 2, 64, 12)):
        c = _case(seed, lengths, h, kvh, dim)
        want = ops.attention_decode(c["q"], c["ks"], c["vs"], c["table"], c["slot"], c["kv_len"], h, kvh,
                                    dim, dim ** -0.5, None, splits)
        # and, independent of any splitting, the plain row-by-row kernel
        pos = (c["kv_len"] - 1).to(torch.int32)
        plain = ops.attention_rowwise(c["q"], c["ks"], c["vs"], c["table"], c["slot"], pos, h, kvh, dim,
                                      dim ** -0.5, None)
        out = torch.empty_like(c["q"])
        _call(lib, c, h, kvh, dim, splits, out=torch.empty_like(c["q"]))      # loads the kernels' code
        with _nothing_else_frees():
            free_before = torch.cuda.mem_get_info()[0]
            rc, got = _call(lib, c, h, kvh, dim, splits, out=out)
            torch.cuda.synchronize()
            free_after = torch.cuda.mem_get_info()[0]
        assert rc == 0, lib.sb_attention_decode_noalloc_message()
        assert free_after == free_before
        assert torch.equal(got, want), "same kernels, same split: the scratch's place must not matter"
        assert torch.allclose(got.float(), plain.float(), **TOL)
    # more scratch than the array holds is refused, with a message that says so, and nothing runs
    big = _case(3, [10] * 64, 32, 8, 128)
    rc, _ = _call(lib, big, 32, 8, 128, 32)
    assert rc == -5
    text = lib.sb_attention_decode_noalloc_message().decode()
    assert "floats of scratch are needed" in text and "1048576" in text
    rc, got = _call(lib, big, 32, 8, 128, 2)
    torch.cuda.synchronize()
    want = ops.attention_decode(big["q"], big["ks"], big["vs"], big["table"], big["slot"], big["kv_len"],
                                32, 8, 128, 128 ** -0.5, None, 2)
    assert rc == 0 and torch.allclose(got.float(), want.float(), **TOL)
