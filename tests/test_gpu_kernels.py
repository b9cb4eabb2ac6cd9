"""Each CUDA kernel alone against a plain torch statement of the same op, at sizes other than the
engine's, with inputs built so that a fault shows (a far key, a window's edge, a page's edge)."""

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": dict(atol=2e-5, rtol=2e-5), "bfloat16": dict(atol=2e-2, rtol=2e-2)}


def dev(t):
    return t.to("cuda")


def rand(*shape, dtype="float32", seed=0, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=gen) * scale).to(DT[dtype])


@pytest.mark.parametrize("dtype", list(DT))
def test_embedding_gathers_rows_and_flags_bad_ids(dtype):
    from starter_b200 import ops

    table = rand(37, 1000, dtype=dtype)
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32)
    out = ops.embedding(dev(ids), dev(table))
    assert torch.equal(out.cpu(), table[ids.long()])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.embedding(dev(torch.tensor([3, 37], dtype=torch.int32)), dev(table), status)
    assert status.item() == 1 and out[1].abs().sum().item() == 0


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("hidden", [24, 1000, 2560, 5121])
def test_rmsnorm_alone_with_the_residual_sum_and_on_chosen_rows(dtype, hidden):
    from starter_b200 import ops

    x, d = rand(9, hidden, dtype=dtype, seed=1), rand(9, hidden, dtype=dtype, seed=2)
    gain = (1 + 0.1 * rand(hidden, seed=3)).to(DT[dtype])
    eps = 1e-5
    want = plain.plain_rms_norm(x, gain, eps)
    assert torch.allclose(ops.rmsnorm(dev(x), dev(gain), eps).cpu().float(), want.float(), **TOL[dtype])
    total = x + d                                   # the sum is rounded to the working type, then normed
    res = dev(x.clone())
    got = ops.rmsnorm(res, dev(gain), eps, delta=dev(d))
    assert torch.equal(res.cpu(), total)
    assert torch.allclose(got.cpu().float(), plain.plain_rms_norm(total, gain, eps).float(), **TOL[dtype])
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    res = dev(x.clone())
    got = ops.rmsnorm(res, dev(gain), eps, delta=dev(d), rows=dev(rows))
    assert torch.equal(res.cpu(), x)                # untouched
    assert torch.allclose(got.cpu().float(), plain.plain_rms_norm(total[rows.long()], gain, eps).float(), **TOL[dtype])
    if dtype == "bfloat16":                         # a gain stored in 32-bit stays 32-bit
        got = ops.rmsnorm(dev(x), dev(gain.float()), eps)
        assert torch.allclose(got.cpu().float(), want.float(), **TOL[dtype])


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("hidden", [24, 1000, 2560, 5128])
def test_rmsnorm_of_many_rows(dtype, hidden):
    """More than 256 rows take the warp-per-row kernel: alone and with the residual sum, a row count
    that does not fill the last block, and the same values as the few-row kernel gives row by row."""
    from starter_b200 import ops

    n = 301
    x, d = rand(n, hidden, dtype=dtype, seed=4), rand(n, hidden, dtype=dtype, seed=5)
    gain = (1 + 0.1 * rand(hidden, seed=6)).to(DT[dtype])
    eps = 1e-6
    got = ops.rmsnorm(dev(x), dev(gain), eps)
    assert torch.allclose(got.cpu().float(), plain.plain_rms_norm(x, gain, eps).float(), **TOL[dtype])
    few = torch.cat([ops.rmsnorm(dev(x[i:i + 100].contiguous()), dev(gain), eps) for i in range(0, n, 100)])
    assert torch.allclose(got.float(), few.float(), **TOL[dtype])
    total = x + d
    res = dev(x.clone())
    got = ops.rmsnorm(res, dev(gain), eps, delta=dev(d))
    assert torch.equal(res.cpu(), total)
    assert torch.allclose(got.cpu().float(), plain.plain_rms_norm(total, gain, eps).float(), **TOL[dtype])
    if dtype == "bfloat16":
        got = ops.rmsnorm(dev(x), dev(gain.float()), eps)
        assert torch.allclose(got.cpu().float(), plain.plain_rms_norm(x, gain, eps).float(), **TOL[dtype])


@pytest.mark.parametrize("dtype", list(DT))
def test_swiglu(dtype):
    from starter_b200 import ops

    gu = rand(5, 2 * 311, dtype=dtype, seed=4, scale=3.0)
    want = plain.plain_swiglu(gu[:, :311], gu[:, 311:])
    assert torch.allclose(ops.swiglu(dev(gu)).cpu().float(), want.float(), **TOL[dtype])


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("rows,n,k", [(1, 7, 96), (2, 301, 100), (3, 64, 2560), (8, 33, 264), (16, 130, 1000),
                                      (17, 70, 96), (130, 257, 77), (200, 1000, 264)])
def test_linear_every_row_count_and_odd_sizes(dtype, rows, n, k):
    from starter_b200 import ops

    x, w = rand(rows, k, dtype=dtype, seed=5), rand(n, k, dtype=dtype, seed=6, scale=0.05)
    want = x.double() @ w.double().t()
    got = ops.linear(dev(x), dev(w))
    assert got.dtype == DT[dtype]
    assert torch.allclose(got.cpu().double(), want, **TOL[dtype])
    got32 = ops.linear(dev(x), dev(w), out_float=True)
    assert got32.dtype == torch.float32
    assert torch.allclose(got32.cpu().double(), want, atol=2e-5 if dtype == "float32" else 2e-3, rtol=1e-3)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("rows", [1, 5, 16, 40])
def test_gated_linear_equals_product_then_swiglu(dtype, rows):
    from starter_b200 import ops

    inner, k = 150, 96
    x, w = rand(rows, k, dtype=dtype, seed=7), rand(2 * inner, k, dtype=dtype, seed=8, scale=0.3)
    gu = (x.double() @ w.double().t()).to(DT[dtype])
    want = plain.plain_swiglu(gu[:, :inner], gu[:, inner:])
    got = ops.linear(dev(x), dev(w), gated=True)
    assert got.shape == (rows, inner)
    assert torch.allclose(got.cpu().float(), want.float(), **TOL[dtype])


def test_a_row_of_the_product_does_not_depend_on_the_other_rows():
    from starter_b200 import ops

    x, w = rand(16, 264, seed=9), rand(50, 264, seed=10)
    full = ops.linear(dev(x), dev(w))
    for rows in (1, 2, 5, 9):
        assert torch.equal(ops.linear(dev(x[:rows]), dev(w)), full[:rows])


def paged(keys, values, n_pages, order):
    """File ``[T, kv_heads, D]`` keys and values of ONE sequence into pages chosen by ``order``."""
    tokens, kv_heads, d = keys.shape
    ks = torch.full((n_pages, kv_heads, 64, d), 7.0, dtype=keys.dtype)   # junk that must never be read
    vs = torch.full((n_pages, kv_heads, 64, d), -7.0, dtype=keys.dtype)
    for t in range(tokens):
        ks[order[t // 64], :, t % 64] = keys[t]
        vs[order[t // 64], :, t % 64] = values[t]
    return ks, vs


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("heads,kv_heads,d", [(4, 2, 16), (6, 2, 48), (5, 5, 128), (8, 1, 256)])
def test_qk_norm_rope_store_files_keys_at_each_tokens_own_place(dtype, heads, kv_heads, d):
    from starter_b200 import ops

    tokens, eps, theta = 11, 1e-5, 1e4
    qkv = rand(tokens, (heads + 2 * kv_heads) * d, dtype=dtype, seed=11)
    qg, kg = ((1 + 0.1 * rand(d, seed=s)).to(DT[dtype]) for s in (12, 13))
    # two sequences: slot 2 continues at position 60 (crossing a page edge), slot 0 starts at 0
    pos = torch.tensor([60, 61, 62, 63, 64, 65, 66, 0, 1, 2, 3], dtype=torch.int32)
    slot = torch.tensor([2] * 7 + [0] * 4, dtype=torch.int32)
    table = torch.tensor([[5, 0, 0], [0, 0, 0], [3, 1, 0]], dtype=torch.int32)
    freqs = plain.plain_rope_tables(theta, d, 128, torch.float32)
    cos32, sin32 = freqs[0][:, : d // 2].contiguous(), freqs[1][:, : d // 2].contiguous()
    ks = torch.zeros(6, kv_heads, 64, d, dtype=DT[dtype], device="cuda")
    vs = torch.zeros_like(ks)
    q = ops.qk_norm_rope_store(dev(qkv), heads, kv_heads, d, dev(qg), dev(kg), eps, dev(cos32), dev(sin32),
                               dev(pos), dev(slot), dev(table), ks, vs)
    cos, sin = (t[pos.long()].to(DT[dtype]) for t in freqs)
    q_in = qkv[:, : heads * d].view(tokens, heads, d)
    k_in = qkv[:, heads * d:(heads + kv_heads) * d].view(tokens, kv_heads, d)
    v_in = qkv[:, (heads + kv_heads) * d:].view(tokens, kv_heads, d)
    q_want = plain.plain_apply_rope(plain.plain_rms_norm(q_in, qg, eps), cos, sin)
    k_want = plain.plain_apply_rope(plain.plain_rms_norm(k_in, kg, eps), cos, sin)
    assert torch.allclose(q.cpu().float().view(tokens, heads, d), q_want.float(), **TOL[dtype])
    ks, vs = ks.cpu(), vs.cpu()
    touched = torch.zeros(6, 64, dtype=torch.bool)
    for t in range(tokens):
        page = table[slot[t], pos[t] // 64].item()
        off = pos[t].item() % 64
        touched[page, off] = True
        assert torch.allclose(ks[page, :, off].float(), k_want[t].float(), **TOL[dtype])
        assert torch.equal(vs[page, :, off], v_in[t])
    untouched = ~touched[:, None, :, None]
    assert (ks * untouched).abs().sum().item() == 0 and (vs * untouched).abs().sum().item() == 0
    # queries alone, nothing written
    q2 = ops.qk_norm_rope_store(dev(qkv[:, : heads * d].contiguous()), heads, kv_heads, d, dev(qg), dev(kg), eps,
                                dev(cos32), dev(sin32), dev(pos), dev(slot), dev(table), None, None,
                                write_cache=False)
    assert torch.equal(q2, q)


def attention_case(dtype, heads, kv_heads, d, lengths, new, window, seed, spike=None):
    """Sequences with ``lengths[i]`` cached tokens of which the last ``new[i]`` are this step's queries.
    Returns what the kernel needs and the plain answer per query row."""
    scale = d ** -0.5
    n_pages, next_page = 40, 0
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    ks = torch.full((n_pages, kv_heads, 64, d), 9.0, dtype=DT[dtype])
    vs = torch.full((n_pages, kv_heads, 64, d), -9.0, dtype=DT[dtype])
    table = torch.zeros(len(lengths), 8, dtype=torch.int32)
    q_rows, slots, poss, wants = [], [], [], []
    for s, (length, n) in enumerate(zip(lengths, new)):
        k = rand(length, kv_heads, d, dtype=dtype, seed=seed + 3 * s)
        v = rand(length, kv_heads, d, dtype=dtype, seed=seed + 3 * s + 1)
        q = rand(length, heads, d, dtype=dtype, seed=seed + 3 * s + 2)
        if spike is not None and spike < length:
            # one far key must win for the last query: align them and make them large
            k[spike] = (q[length - 1, :: heads // kv_heads][:kv_heads] * 4).to(DT[dtype])
        for p in range((length + 63) // 64):
            table[s, p] = perm[next_page]
            next_page += 1
        for t in range(length):
            ks[table[s, t // 64], :, t % 64] = k[t]
            vs[table[s, t // 64], :, t % 64] = v[t]
        want = plain.plain_attention(q, k, v, scale, window)
        for t in range(length - n, length):
            q_rows.append(q[t].reshape(-1))
            slots.append(s)
            poss.append(t)
            wants.append(want[t].reshape(-1))
    return dict(q=torch.stack(q_rows), ks=ks, vs=vs, table=table,
                slot=torch.tensor(slots, dtype=torch.int32), pos=torch.tensor(poss, dtype=torch.int32),
                want=torch.stack(wants), scale=scale, q_start=None)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("heads,kv_heads,d,window", [(4, 2, 16, None), (6, 2, 48, 5), (8, 8, 128, None),
                                                    (8, 1, 64, 70), (3, 1, 256, None)])
def test_attention_rowwise(dtype, heads, kv_heads, d, window):
    from starter_b200 import ops

    c = attention_case(dtype, heads, kv_heads, d, lengths=[130, 1, 64, 200], new=[130, 1, 3, 1],
                       window=window, seed=20, spike=2)
    got = ops.attention_rowwise(dev(c["q"]), dev(c["ks"]), dev(c["vs"]), dev(c["table"]), dev(c["slot"]),
                                dev(c["pos"]), heads, kv_heads, d, c["scale"], window)
    assert torch.allclose(got.cpu().float(), c["want"].float(), **TOL[dtype])


def test_sampling_greedy_ties_and_seeded_draws():
    from starter_b200 import ops
    from starter_b200.sampling import gumbel_noise, request_key

    logits = torch.zeros(3, 1000)
    logits[0, [400, 7, 900]] = 2.0          # equal maxima: the lowest index wins
    logits[1, 999] = 1.0
    logits[2] = -1.0
    logits[2, 0] = float("nan")
    assert ops.sample(dev(logits)).tolist() == [7, 999, 1]
    rows = rand(6, 5003, seed=30, scale=2.0)
    temps = [0.0, 0.7, 1.5, 0.7, 0.0, 3.0]
    keys = [request_key(9, i) for i in range(6)]
    poss = [3, 3, 8, 4, 1, 0]
    got = ops.sample(dev(rows), dev(torch.tensor(temps)), dev(torch.tensor(np.asarray(keys, dtype=np.uint32).view(np.int32))),
                     dev(torch.tensor(poss, dtype=torch.int32))).tolist()
    for i in range(6):
        assert got[i] == plain.plain_select(rows[i].numpy(), temps[i], keys[i], poss[i])
    nan = torch.full((1, 10), float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert ops.sample(dev(nan), status=status).tolist() == [0] and status.item() == 2


def test_refusals_name_the_size():
    from starter_b200 import ops

    with pytest.raises(ops.KernelError, match="CUDA tensor"):
        ops.rmsnorm(torch.zeros(2, 4), torch.ones(4), 1e-6)
    with pytest.raises(ops.KernelError, match="head_dim"):
        ops.attention_rowwise(dev(torch.zeros(1, 2 * 320)), dev(torch.zeros(1, 1, 64, 320)),
                              dev(torch.zeros(1, 1, 64, 320)), dev(torch.zeros(1, 1, dtype=torch.int32)),
                              dev(torch.zeros(1, dtype=torch.int32)), dev(torch.zeros(1, dtype=torch.int32)),
                              2, 1, 320, 1.0)
    with pytest.raises(ops.KernelError, match="contiguous"):
        ops.linear(dev(torch.zeros(4, 8)).t(), dev(torch.zeros(3, 4)))
    with pytest.raises(ops.KernelError, match="width"):
        ops.linear(dev(torch.zeros(4, 8)), dev(torch.zeros(3, 9)))


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("heads,kv_heads,d,window,splits", [
    (4, 2, 16, None, 1), (6, 2, 32, 5, 3), (8, 8, 128, None, 4), (8, 1, 64, 70, 2), (3, 1, 256, None, 7),
    (32, 8, 128, None, None), (10, 2, 64, 64, 16)])
def test_attention_decode_split_over_keys(dtype, heads, kv_heads, d, window, splits):
    """One query per row; lengths 1 (a single key), 64 and 65 (a page's edge), 200; more splits than
    pages (empty parts must drop out); a far key made to win; the window's first key."""
    from starter_b200 import ops

    if not ops.decode_attention_takes(d, DT[dtype]):
        with pytest.raises(ops.KernelError, match="head_dim"):
            ops.attention_decode(dev(torch.zeros(1, heads * d, dtype=DT[dtype])), None, None, None, None, None,
                                 heads, kv_heads, d, 1.0)
        return
    lengths = [130, 1, 64, 65, 200]
    c = attention_case(dtype, heads, kv_heads, d, lengths=lengths, new=[1] * 5, window=window, seed=40, spike=3)
    kv_len = torch.tensor(lengths, dtype=torch.int32)
    rows = torch.arange(5, dtype=torch.int32)
    got = ops.attention_decode(dev(c["q"]), dev(c["ks"]), dev(c["vs"]), dev(c["table"]), dev(rows), dev(kv_len),
                               heads, kv_heads, d, c["scale"], window, splits)
    assert torch.allclose(got.cpu().float(), c["want"].float(), **TOL[dtype])
    plain_kernel = ops.attention_rowwise(dev(c["q"]), dev(c["ks"]), dev(c["vs"]), dev(c["table"]), dev(c["slot"]),
                                         dev(c["pos"]), heads, kv_heads, d, c["scale"], window)
    assert torch.allclose(got.cpu().float(), plain_kernel.cpu().float(), **TOL[dtype])


@pytest.mark.parametrize("gain_dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("heads,kv_heads,d,window,splits,norm,rope", [
    (4, 2, 16, None, 1, True, True), (6, 2, 32, 5, 3, True, False), (32, 8, 128, None, None, True, True),
    (8, 1, 64, 70, 2, False, True), (40, 2, 64, None, 16, True, True)])
def test_attention_decode_from_qkv_equals_the_separate_kernels(heads, kv_heads, d, window, splits, norm, rope, gain_dtype):
    """The decode kernel that norms, rotates and files the new key and value itself gives the same
    bits, in its output and in the cache, as qk_norm_rope_store followed by attention_decode: lengths 1
    (the new token is the only key), 64 and 65 (it ends or starts a page), 130, 200; scattered pages;
    also a layer that only reads a cache (queries alone)."""
    from starter_b200 import ops

    lengths = [130, 1, 64, 65, 200]
    c = attention_case("bfloat16", heads, kv_heads, d, lengths=lengths, new=[1] * 5, window=window, seed=70)
    kv_len = dev(torch.tensor(lengths, dtype=torch.int32))
    slots = dev(torch.arange(5, dtype=torch.int32))
    pos = dev(torch.tensor([n - 1 for n in lengths], dtype=torch.int32))
    qkv = dev(rand(5, (heads + 2 * kv_heads) * d, dtype="bfloat16", seed=71))
    gq = dev(1 + rand(d, dtype=gain_dtype, seed=72, scale=0.2)) if norm else None
    gk = dev(1 + rand(d, dtype=gain_dtype, seed=73, scale=0.2)) if norm else None
    cos = dev(torch.cos(rand(256, d // 2, seed=74, scale=3.0))) if rope else None
    sin = dev(torch.sin(rand(256, d // 2, seed=74, scale=3.0))) if rope else None
    table = dev(c["table"])
    for write_cache in (True, False):
        x = qkv if write_cache else qkv[:, : heads * d].contiguous()
        ks_a, vs_a, ks_b, vs_b = dev(c["ks"]), dev(c["vs"]), dev(c["ks"]), dev(c["vs"])
        q = ops.qk_norm_rope_store(x, heads, kv_heads, d, gq, gk, 1e-5, cos, sin, pos, slots, table, ks_a, vs_a,
                                   write_cache=write_cache)
        want = ops.attention_decode(q, ks_a, vs_a, table, slots, kv_len, heads, kv_heads, d, c["scale"], window, splits)
        got = ops.attention_decode_qkv(x, ks_b, vs_b, table, slots, kv_len, heads, kv_heads, d, c["scale"], window,
                                       gq, gk, 1e-5, cos, sin, write_cache=write_cache, n_splits=splits)
        assert torch.equal(got, want)
        assert torch.equal(ks_a, ks_b) and torch.equal(vs_a, vs_b)
        if write_cache:
            assert not torch.equal(ks_b.cpu(), c["ks"])      # the new keys went in


@pytest.mark.parametrize("rows,n,k,gated,bm,splits", [
    (1, 128, 64, False, 16, 1), (8, 256, 512, False, 16, 2), (5, 300, 1000, False, None, None),
    (16, 2560, 4096, False, None, None), (64, 1000, 2560, False, None, None), (3, 200, 264, False, 16, 5),
    (64, 2560, 4096, False, 64, 8), (40, 384, 1024, True, 64, 4),
    (8, 1216, 2560, True, None, None), (33, 640, 2568, True, None, 3), (1, 64, 8, True, 16, 1),
    (200, 520, 1000, False, None, None), (600, 777, 264, False, 256, 1), (257, 130, 72, False, 128, 2)])
def test_tensor_core_product(rows, n, k, gated, bm, splits):
    """The tcgen05 product at sizes that are no multiples of its tiles, with and without splitting k,
    plain and gated, bfloat16 and float32 results; and twice, since it keeps counters between calls."""
    from starter_b200 import ops

    x = rand(rows, k, dtype="bfloat16", seed=50)
    w = rand(n * (2 if gated else 1), k, dtype="bfloat16", seed=51, scale=0.05)
    ref = x.double() @ w.double().t()
    if gated:
        gu = ref.to(torch.bfloat16)
        ref = plain.plain_swiglu(gu[:, :n], gu[:, n:]).double()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):
        got = ops.linear_tensor_core(dev(x), dev(w), gated=gated, bm=bm, splits=splits, status=status)
        assert got.shape == (rows, n) and got.dtype == torch.bfloat16
        assert torch.allclose(got.cpu().double(), ref, atol=2e-2, rtol=2e-2)
    if not gated:
        got32 = ops.linear_tensor_core(dev(x), dev(w), out_float=True, bm=bm, splits=splits, status=status)
        assert torch.allclose(got32.cpu().double(), ref, atol=1e-4, rtol=1e-4)
        again = ops.linear_tensor_core(dev(x), dev(w), out_float=True, bm=bm, splits=splits, status=status)
        assert torch.equal(got32, again)            # parts are added in split order, whoever ends last
    assert status.item() == 0


def test_a_wait_in_the_prompt_attention_that_runs_out_is_reported():
    """The tcgen05 prompt attention with half of one step's values left out on purpose: the wait on
    them gives up after 2 ms, every block returns, bit 16 of the status word is set; the same call
    without the gap is right afterwards."""
    from starter_b200 import ops
    from starter_b200.engine.runner import ModelRunner

    heads, kv_heads, d = 4, 2, 128
    lengths = [300, 260]
    c = attention_case("bfloat16", heads, kv_heads, d, lengths=lengths, new=lengths, window=None, seed=88)
    q_start = [0, lengths[0]]
    tiles = [(i, f) for i in range(2) for f in range(0, lengths[i], 64)]
    ints = lambda v: dev(torch.tensor(v, dtype=torch.int32))
    status = dev(torch.zeros(1, dtype=torch.int32))
    args = (dev(c["q"]), dev(c["ks"]), dev(c["vs"]), dev(c["table"]), ints([0, 1]), ints(q_start), ints(lengths),
            ints(lengths), ints([t[0] for t in tiles]), ints([t[1] for t in tiles]), heads, kv_heads, d, c["scale"], None)
    ops.attention_prefill(*args, status=status, kernel="tcgen05", withhold=(0, 2_000_000))
    torch.cuda.synchronize()
    assert status.item() == 16
    holder = ModelRunner.__new__(ModelRunner)
    holder.status = status
    with pytest.raises(RuntimeError, match="prefill attention kernel ran out of time"):
        holder.check_status()
    got = ops.attention_prefill(*args, status=status, kernel="tcgen05")
    assert status.item() == 0
    assert torch.allclose(got.cpu().float(), c["want"].float(), atol=2e-2, rtol=2e-2)


def test_a_wait_in_the_decode_attention_that_runs_out_is_reported():
    """The CUDA-core decode attention (the float32 path's) with one page's values left out on purpose:
    the wait on that page gives up after 2 ms, the kernel returns, bit 8 of the status word is set; the
    same call without the gap is right afterwards."""
    from starter_b200 import ops
    from starter_b200.engine.runner import ModelRunner

    heads, kv_heads, d = 4, 2, 32
    lengths = [200, 130]
    c = attention_case("float32", heads, kv_heads, d, lengths=lengths, new=[1, 1], window=None, seed=77)
    status = dev(torch.zeros(1, dtype=torch.int32))
    args = (dev(c["q"]), dev(c["ks"]), dev(c["vs"]), dev(c["table"]), dev(c["slot"]),
            dev(torch.tensor(lengths, dtype=torch.int32)), heads, kv_heads, d, c["scale"], None)
    ops.attention_decode(*args, n_splits=1, status=status, withhold=(1, 2_000_000))
    torch.cuda.synchronize()
    assert status.item() == 8
    holder = ModelRunner.__new__(ModelRunner)
    holder.status = status
    with pytest.raises(RuntimeError, match="decode attention kernel ran out of time"):
        holder.check_status()
    got = ops.attention_decode(*args, n_splits=1, status=status)
    assert status.item() == 0
    assert torch.allclose(got.cpu(), c["want"], atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("rows,n,k,gated,splits,stage", [(8, 256, 512, False, 1, 0), (8, 384, 1024, False, 4, 1),
                                                       (16, 128, 768, True, 2, 2)])
def test_a_wait_in_the_tensor_core_product_that_runs_out_is_reported(rows, n, k, gated, splits, stage):
    """One activation copy of every block is left out on purpose (an entry point made for this), so
    the stage it belongs to never completes: the wait on it gives up after 2 ms, the kernel returns,
    the status word says so and ``check_status`` turns it into an error.  The device stays usable:
    the same product, run normally afterwards, is right."""
    from starter_b200 import ops
    from starter_b200.engine.runner import ModelRunner

    x = rand(rows, k, dtype="bfloat16", seed=60)
    w = rand(n * (2 if gated else 1), k, dtype="bfloat16", seed=61, scale=0.05)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.linear_tensor_core(dev(x), dev(w), gated=gated, bm=16, splits=splits, stages=4, status=status,
                           withhold=(stage, 2_000_000))
    torch.cuda.synchronize()
    assert status.item() == 4
    holder = ModelRunner.__new__(ModelRunner)         # check_status needs nothing but the word
    holder.status = status
    with pytest.raises(RuntimeError, match="tensor-core product ran out of time"):
        holder.check_status()
    assert status.item() == 0
    got = ops.linear_tensor_core(dev(x), dev(w), gated=gated, bm=16, splits=splits, stages=4, status=status)
    ref = x.double() @ w.double().t()
    if gated:
        gu = ref.to(torch.bfloat16)
        ref = plain.plain_swiglu(gu[:, :n], gu[:, n:]).double()
    assert torch.allclose(got.cpu().double(), ref, atol=2e-2, rtol=2e-2) and status.item() == 0


@pytest.mark.parametrize("rows,n,k,gated,bn,pairs", [
    (256, 256, 128, False, 256, 1), (512, 512, 192, False, 0, 0), (300, 200, 72, False, 0, 0),
    (300, 320, 136, False, 160, 0), (1, 64, 8, False, 64, 0), (700, 777, 264, False, 192, 3),
    (256, 128, 128, True, 256, 1), (700, 448, 264, True, 0, 0), (333, 192, 200, True, 128, 0),
    (65, 100, 40, True, 64, 0), (2048, 2560, 1024, False, 0, 0), (1100, 1216, 2560, True, 0, 0),
    (4500, 300, 136, False, 0, 0), (4400, 128, 72, True, 0, 5)])
def test_prompt_product(rows, n, k, gated, bn, pairs):
    """The CTA-pair product for many rows at sizes that are no multiples of its tiles (rows past the
    end of a 256-row tile, widths past the end of a weight tile, a k that ends inside a 64-wide
    block), every tile width, one pair or all of them (so that a pair works through several tiles
    and both accumulators), more row tiles than one group holds, plain and gated; twice, and bit-equal both times."""
    from starter_b200 import ops

    x = rand(rows, k, dtype="bfloat16", seed=52)
    w = rand(n * (2 if gated else 1), k, dtype="bfloat16", seed=53, scale=0.05)
    ref = x.double() @ w.double().t()
    if gated:
        gu = ref.to(torch.bfloat16)
        ref = plain.plain_swiglu(gu[:, :n], gu[:, n:]).double()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.linear_prompt(dev(x), dev(w), gated=gated, bn=bn, pairs=pairs, status=status)
    assert got.shape == (rows, n) and got.dtype == torch.bfloat16
    assert torch.allclose(got.cpu().double(), ref, atol=2e-2, rtol=2e-2)
    again = ops.linear_prompt(dev(x), dev(w), gated=gated, bn=bn, pairs=pairs, status=status)
    assert torch.equal(got, again)
    assert status.item() == 0


@pytest.mark.parametrize("rows,n,k,bn", [(512, 256, 128, 0), (700, 777, 264, 192), (300, 200, 72, 0), (2048, 2560, 512, 0)])
def test_prompt_product_adds_onto_the_residual_stream(rows, n, k, bn):
    """The residual epilogue: the stream becomes round(stream + round(product)) in place, exactly
    what the product followed by a separate bfloat16 add gives; and ``ops.linear`` takes the offer
    only where that kernel runs."""
    from starter_b200 import ops

    x = dev(rand(rows, k, dtype="bfloat16", seed=64))
    w = dev(rand(n, k, dtype="bfloat16", seed=65, scale=0.05))
    stream = dev(rand(rows, n, dtype="bfloat16", seed=66))
    product = ops.linear_prompt(x, w, bn=bn)
    want = (stream.float() + product.float()).to(torch.bfloat16)
    got = stream.clone()
    back = ops.linear_prompt(x, w, bn=bn, residual=got)
    assert back is got and torch.equal(got, want)
    offered = stream.clone()
    answer = ops.linear(x, w, add_to=offered)
    if rows >= ops.PROMPT_MIN_ROWS:
        assert answer is ops.ADDED and torch.equal(offered, want)
    else:
        assert torch.equal(offered, stream) and torch.allclose(answer.float(), product.float(), atol=2e-2, rtol=2e-2)
    with pytest.raises(ops.KernelError, match="residual"):
        ops.linear_prompt(x, w, residual=stream[:, :-8].contiguous())


def test_prompt_product_is_the_few_row_product_row_by_row():
    """A prompt's rows through the CTA-pair kernel and the same rows, 16 at a time, through the
    kernel that decoding uses: the same sums in another order, so equal to rounding (and the gated
    epilogue rounds at the same places)."""
    from starter_b200 import ops

    x = dev(rand(600, 520, dtype="bfloat16", seed=54))
    for gated in (False, True):
        w = dev(rand(384 * (2 if gated else 1), 520, dtype="bfloat16", seed=55, scale=0.05))
        many = ops.linear_prompt(x, w, gated=gated)
        few = torch.cat([ops.linear_tensor_core(x[i:i + 16].contiguous(), w, gated=gated) for i in range(0, 600, 16)])
        assert torch.allclose(many.float(), few.float(), atol=2e-2, rtol=2e-2)
        assert (many != few).float().mean().item() < 0.05


def test_linear_sends_each_row_count_to_its_kernel(monkeypatch):
    """``ops.linear`` in bfloat16: the tcgen05 product up to TENSOR_CORE_MAX_ROWS rows, the CTA-pair
    product from PROMPT_MIN_ROWS rows on, and both agree with the plain product."""
    from starter_b200 import ops

    taken = []
    few, many = ops.linear_tensor_core, ops.linear_prompt
    monkeypatch.setattr(ops, "linear_tensor_core", lambda *a, **k: (taken.append("few"), few(*a, **k))[1])
    monkeypatch.setattr(ops, "linear_prompt", lambda *a, **k: (taken.append("many"), many(*a, **k))[1])
    w = rand(200, 264, dtype="bfloat16", seed=57, scale=0.05)
    for rows, want in ((ops.TENSOR_CORE_MAX_ROWS, "few"), (ops.PROMPT_MIN_ROWS, "many"), (ops.PROMPT_MIN_ROWS + 77, "many")):
        x = rand(rows, 264, dtype="bfloat16", seed=56)
        got = ops.linear(dev(x), dev(w))
        assert taken[-1] == want
        assert torch.allclose(got.cpu().double(), x.double() @ w.double().t(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("rows,n,k,gated,kblock", [(256, 256, 512, False, 0), (600, 384, 1024, True, 3)])
def test_a_wait_in_the_prompt_product_that_runs_out_is_reported(rows, n, k, gated, kblock):
    """One weight copy of every first CTA is left out on purpose (an entry point made for this): the
    stage never fills, the waits of both CTAs of the pair give up after 2 ms, the kernel returns with
    its tensor memory freed, the status word says so; the same product, run normally afterwards, is
    right."""
    from starter_b200 import ops
    from starter_b200.engine.runner import ModelRunner

    x = rand(rows, k, dtype="bfloat16", seed=62)
    w = rand(n * (2 if gated else 1), k, dtype="bfloat16", seed=63, scale=0.05)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.linear_prompt(dev(x), dev(w), gated=gated, status=status, withhold=(kblock, 2_000_000))
    torch.cuda.synchronize()
    assert status.item() == 4
    holder = ModelRunner.__new__(ModelRunner)
    holder.status = status
    with pytest.raises(RuntimeError, match="tensor-core product ran out of time"):
        holder.check_status()
    assert status.item() == 0
    got = ops.linear_prompt(dev(x), dev(w), gated=gated, status=status)
    ref = x.double() @ w.double().t()
    if gated:
        gu = ref.to(torch.bfloat16)
        ref = plain.plain_swiglu(gu[:, :n], gu[:, n:]).double()
    assert torch.allclose(got.cpu().double(), ref, atol=2e-2, rtol=2e-2) and status.item() == 0


@pytest.mark.parametrize("heads,kv_heads,d,window", [(4, 2, 16, None), (6, 2, 32, 5), (8, 8, 128, None),
                                                    (8, 1, 64, 70), (32, 8, 128, None), (4, 4, 64, 64),
                                                    (6, 3, 128, 130)])
@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
def test_attention_prefill_many_tokens_per_sequence(heads, kv_heads, d, window, kernel):
    """Both prefill kernels (mma.sync tiles of 64 queries; tcgen05 tiles of 128 for head sizes 64 and
    128).  Whole prompts, a chunk that continues a sequence (its first query is not at position 0), one
    query, lengths at and next to the tile and page edges, scattered pages, a far key made to win."""
    from starter_b200 import ops

    if kernel == "tcgen05" and d not in ops.PREFILL_TC_HEAD_DIMS:
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128")
    status = dev(torch.zeros(1, dtype=torch.int32))
    lengths, new = [130, 1, 64, 200, 65, 300, 450], [130, 1, 3, 77, 65, 129, 450]
    c = attention_case("bfloat16", heads, kv_heads, d, lengths=lengths, new=new, window=window, seed=60, spike=2)
    q_start = [sum(new[:i]) for i in range(len(new))]
    tiles = [(i, f) for i in range(len(new)) for f in range(0, new[i], 64)]
    ints = lambda v: dev(torch.tensor(v, dtype=torch.int32))
    got = ops.attention_prefill(dev(c["q"]), dev(c["ks"]), dev(c["vs"]), dev(c["table"]), ints(list(range(len(new)))),
                                ints(q_start), ints(new), ints(lengths), ints([t[0] for t in tiles]),
                                ints([t[1] for t in tiles]), heads, kv_heads, d, c["scale"], window,
                                status=status, kernel=kernel)
    assert status.item() == 0
    assert torch.allclose(got.cpu().float(), c["want"].float(), atol=2e-2, rtol=2e-2)
    if kernel == "tcgen05":
        # the kernel's own work list (one entry per block of 256 queries): the same blocks, none idle
        blocks = [(i, f) for i in range(len(new)) for f in range(0, new[i], 256)]
        again = ops.attention_prefill(dev(c["q"]), dev(c["ks"]), dev(c["vs"]), dev(c["table"]),
                                      ints(list(range(len(new)))), ints(q_start), ints(new), ints(lengths),
                                      ints([t[0] for t in tiles]), ints([t[1] for t in tiles]), heads, kv_heads, d,
                                      c["scale"], window, status=status, kernel=kernel,
                                      blocks=(ints([b[0] for b in blocks]), ints([b[1] for b in blocks])))
        assert torch.equal(again, got) and status.item() == 0
