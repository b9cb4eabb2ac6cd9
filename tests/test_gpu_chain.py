"""Chains of few-row projections and row norms in one persistent kernel (csrc/dense_chain.cu) against
the same operations run one kernel at a time, and against plain torch."""

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def rand(*shape, seed=0, scale=1.0, dtype=torch.bfloat16):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=gen) * scale).to(dtype).cuda()


def close(got, want, what, tol=2e-2):
    got, want = got.float().cpu(), want.float().cpu()
    scale = want.abs().max().item()
    err = (got - want).abs().max().item()
    assert err <= tol * scale, f"{what}: off by {err:.3e} of {scale:.3e}"


def layer_tensors(hidden, q_size, inter, qkv_size, seed, gain_dtype=torch.bfloat16):
    s = 0.7 / hidden ** 0.5
    return dict(
        o=rand(hidden, q_size, seed=seed, scale=0.7 / q_size ** 0.5), gate_up=rand(2 * inter, hidden, seed=seed + 1, scale=s),
        down=rand(hidden, inter, seed=seed + 2, scale=0.7 / inter ** 0.5), qkv=rand(qkv_size, hidden, seed=seed + 3, scale=s),
        g1=(1 + 0.1 * rand(hidden, seed=seed + 4, dtype=torch.float32)).to(gain_dtype),
        g2=(1 + 0.1 * rand(hidden, seed=seed + 5, dtype=torch.float32)).to(gain_dtype))


def one_by_one(ops, t, attn, residual, eps):
    """The chain's operations as separate kernels; returns (qkv, residual after both sums, act)."""
    residual = residual.clone()
    o = ops.linear(attn, t["o"])
    m = ops.rmsnorm(residual, t["g2"], eps, delta=o)
    act = ops.linear(m, t["gate_up"], gated=True)
    d = ops.linear(act, t["down"])
    n = ops.rmsnorm(residual, t["g1"], eps, delta=d)
    return ops.linear(n, t["qkv"]), residual, act


def as_chain(ops, t, attn, residual, eps, status):
    residual = residual.clone()
    chain = ops.OpenChain(attn.shape[0], attn.device, status)
    o = chain.linear(attn, t["o"])
    m = chain.add_norm(residual, o, t["g2"], eps)
    act = chain.linear(m, t["gate_up"], gated=True)
    d = chain.linear(act, t["down"])
    n = chain.add_norm(residual, d, t["g1"], eps)
    qkv = chain.linear(n, t["qkv"])
    return ops.resolve(qkv), residual, ops.resolve(act)


@pytest.mark.parametrize("gain_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,hidden,q_size,inter,qkv_size", [
    (8, 2560, 4096, 9728, 6144), (1, 2560, 4096, 9728, 6144), (64, 2560, 4096, 9728, 6144),
    (33, 1024, 768, 1408, 1280), (16, 96, 192, 192, 200), (5, 264, 72, 64, 136), (17, 5120, 5120, 17408, 7168)])
def test_a_layer_chain_equals_its_operations_one_by_one(rows, hidden, q_size, inter, qkv_size, gain_dtype):
    from starter_b200 import ops

    t = layer_tensors(hidden, q_size, inter, qkv_size, 10, gain_dtype)
    attn = rand(rows, q_size, seed=1)
    residual = rand(rows, hidden, seed=2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    want_qkv, want_res, want_act = one_by_one(ops, t, attn, residual, 1e-6)
    got_qkv, got_res, got_act = as_chain(ops, t, attn, residual, 1e-6, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    close(got_act, want_act, "gated activations")
    close(got_res, want_res, "residual stream after two sums")
    close(got_qkv, want_qkv, "the next projection")
    # and against plain torch in double precision with the roundings of the formulas
    def r(x):
        return x.to(torch.bfloat16).double()
    a, res = attn.double().cpu(), residual.double().cpu()
    w = {k: v.double().cpu() for k, v in t.items()}
    res = r(res + r(a @ w["o"].t()))
    m = plain.plain_rms_norm(res.to(torch.bfloat16), t["g2"].cpu(), 1e-6).double()
    gu = r(m @ w["gate_up"].t())
    act = r(plain.plain_swiglu(gu[:, :inter].to(torch.bfloat16), gu[:, inter:].to(torch.bfloat16)))
    res = r(res + r(act @ w["down"].t()))
    n = plain.plain_rms_norm(res.to(torch.bfloat16), t["g1"].cpu(), 1e-6).double()
    close(got_qkv, r(n @ w["qkv"].t()), "the next projection, against plain torch", tol=3e-2)
    # the same chain again: the same bits (partial tiles are summed in a fixed order)
    again_qkv, again_res, _ = as_chain(ops, t, attn, residual, 1e-6, status)
    assert torch.equal(again_qkv, got_qkv) and torch.equal(again_res, got_res)
    assert status.item() == 0


def test_chains_of_other_shapes_and_what_a_chain_refuses():
    from starter_b200 import ops

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = rand(3, 264, seed=3)
    w = rand(200, 264, seed=4, scale=0.05)
    gain = (1 + 0.1 * rand(264, seed=5, dtype=torch.float32)).to(torch.bfloat16)
    # a norm of a tensor alone, then a projection
    chain = ops.OpenChain(3, x.device, status)
    n = chain.add_norm(x, None, gain, 1e-5)
    y = ops.resolve(chain.linear(n, w))
    close(y, ops.linear(ops.rmsnorm(x, gain, 1e-5), w), "norm alone, then a projection")
    # a delta from outside; the sum is written back
    res, delta = rand(3, 264, seed=6), rand(3, 264, seed=7)
    mine = res.clone()
    chain = ops.OpenChain(3, x.device, status)
    n = chain.add_norm(mine, delta, gain, 1e-5)
    y = ops.resolve(chain.linear(n, w))
    theirs = res.clone()
    want = ops.linear(ops.rmsnorm(theirs, gain, 1e-5, delta=delta), w)
    close(y, want, "sum with an outside delta")
    assert torch.equal(mine, theirs)
    # a single projection, a value read twice, and a second chain started from a value of the first
    chain = ops.OpenChain(3, x.device, status)
    a = chain.linear(x, w)
    b = chain.linear(a, rand(136, 200, seed=8, scale=0.05))
    c = chain.linear(a, rand(72, 200, seed=9, scale=0.05))
    other = ops.OpenChain(3, x.device, status)
    d = other.linear(b, rand(64, 136, seed=11, scale=0.05))
    close(ops.resolve(d), ops.linear(ops.linear(ops.linear(x, w), rand(136, 200, seed=8, scale=0.05)),
                                     rand(64, 136, seed=11, scale=0.05)), "a chain fed by another chain")
    close(ops.resolve(c), ops.linear(ops.linear(x, w), rand(72, 200, seed=9, scale=0.05)), "a value read twice")
    torch.cuda.synchronize()
    assert status.item() == 0
    assert not ops.chain_takes_linear(rand(65, 64), rand(64, 64), False)          # too many rows
    assert not ops.chain_takes_linear(rand(4, 60), rand(64, 60), False)           # k no multiple of 8
    assert not ops.chain_takes_linear(rand(4, 64), rand(2 * 96, 64), True)        # gated width no multiple of 64
    assert not ops.chain_takes_linear(rand(4, 64, dtype=torch.float32), rand(64, 64, dtype=torch.float32), False)
    with pytest.raises(ops.KernelError):
        ops.OpenChain(3, x.device, status).linear(rand(4, 264), w)                # rows differ from the chain's
