"""The fused backward (``kfa_bwd_fused``: dK, dV and dQ from one P and one dS per tile pair, dQ through
fp32 reduce-adds) against the split, bit-reproducible kernels (``kfa_bwd``) and the fp64 oracle.

Both paths feed the tensor cores the same rounded operands; they differ only in the order of fp32
additions (dQ: atomic adds in whatever order the CTAs get there; dK, dV: the fused kernel walks the query
tiles starting at a different tile per key tile). So every gradient must agree with the split kernels' to
``rel_err < 1e-3``, the tolerance the reference uses for its own run-to-run dQ comparison (KohakuFA
tests/test_attention.py:347-358), and dK, dV must repeat bit for bit from run to run."""

import ctypes

import pytest
import torch

from kohakufa_b200 import _lib, attention
from kohakufa_b200.op import attention_fwd_op
from oracle import reference as oracle

pytestmark = pytest.mark.gpu


def make(batch, heads, kv_heads, s_q, s_kv, dim, dtype, seed, std=1.0):
    gen = torch.Generator().manual_seed(seed)

    def proj(h, s):
        return (torch.randn(batch, s, h, dim, generator=gen) * std).to(dtype).cuda().transpose(1, 2)

    return proj(heads, s_q), proj(kv_heads, s_kv), proj(kv_heads, s_kv), proj(heads, s_q)


def backward_both(q, k, v, dout, scale, block):
    """(dq, dk, dv) of the split and of the fused entry points, on the same forward results."""
    lib = _lib.load()
    out, lse = attention_fwd_op(q, k, v, scale, block)
    like = lambda t: t.new_empty(t.shape[0], t.shape[2], t.shape[1], t.shape[3]).transpose(1, 2)  # noqa: E731
    batch, heads, s_q, dim = q.shape
    stats = q.new_empty(lib.kfa_bwd_stats_bytes(batch, heads, s_q) // 4, dtype=torch.float32)
    acc = q.new_empty(lib.kfa_bwd_dq_acc_bytes(batch, heads, s_q, dim) // 4, dtype=torch.float32)
    acc.fill_(float("nan"))  # the call has to clear what it uses
    code, word, stream = _lib.dtype_code(q.dtype), _lib.status_word(q.device).data_ptr(), _lib.stream_ptr(q.device)
    ins = [ctypes.byref(_lib.tensor4(t)) for t in (q, k, v, out, dout)]
    split = [like(q), like(k), like(v)]
    fused = [like(q), like(k), like(v)]
    for g in fused:
        g.fill_(float("nan"))
    _lib.check(lib.kfa_bwd(*ins, lse.data_ptr(), stats.data_ptr(), *(ctypes.byref(_lib.tensor4(t)) for t in split),
                           scale, block, code, word, stream))  # fmt: skip
    _lib.check(lib.kfa_bwd_fused(*ins, lse.data_ptr(), stats.data_ptr(), acc.data_ptr(),
                                 *(ctypes.byref(_lib.tensor4(t)) for t in fused), scale, block, code, word, stream))  # fmt: skip
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, f"a kernel wait timed out: status {_lib.device_status()}"
    return out, split, fused


CASES = [  # batch, heads, kv_heads, s_q, s_kv, dim, dtype, block
    (1, 1, 1, 128, 128, 64, torch.float16, 0),
    (1, 1, 1, 128, 128, 128, torch.bfloat16, 0),
    (2, 2, 2, 256, 256, 64, torch.float16, 1),
    (2, 2, 2, 384, 384, 128, torch.bfloat16, 1),
    (1, 3, 3, 201, 201, 64, torch.float16, 0),
    (1, 2, 2, 1000, 1000, 128, torch.float16, 1),
    (1, 2, 2, 600, 600, 64, torch.bfloat16, 24),
    (1, 2, 2, 600, 600, 128, torch.float16, 257),
    (1, 2, 2, 300, 517, 64, torch.float16, 1),
    (1, 2, 2, 517, 300, 128, torch.bfloat16, 1),
    (1, 2, 2, 130, 700, 128, torch.float16, 128),
    (2, 4, 2, 333, 333, 64, torch.float16, 1),
    (1, 8, 1, 260, 260, 128, torch.bfloat16, 0),
    (1, 2, 2, 2048, 2048, 128, torch.bfloat16, 1),
    (1, 2, 2, 2048, 2048, 64, torch.float16, 256),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(str(x).replace("torch.", "") for x in c))
def test_fused_matches_split_and_oracle(case):
    batch, heads, kv_heads, s_q, s_kv, dim, dtype, block = case
    q, k, v, dout = make(batch, heads, kv_heads, s_q, s_kv, dim, dtype, seed=s_q + dim + block)
    scale = dim**-0.5
    out, split, fused = backward_both(q, k, v, dout, scale, block)
    assert all(bool(torch.isfinite(g).all()) for g in fused)
    for name, f, s in zip(("dQ", "dK", "dV"), fused, split):
        err = oracle.rel_l2(f, s) if float(s.abs().max()) > 0 else float(f.abs().max())
        assert err < 1e-3, f"{name}: {err:.3e} away from the split kernel's"
    want = oracle.attention_fp64(q, k, v, dout, scale, block=block, groups=heads // kv_heads)
    tol = 5e-3 if dtype == torch.float16 else 2e-2
    for name, g, w in zip(("dq", "dk", "dv"), fused, want[1:]):
        if float(w.abs().max()) == 0.0:
            assert float(g.abs().max()) < 1e-4, name
        else:
            assert oracle.metrics(g, w)["rel_err"] < tol, (name, oracle.metrics(g, w))


def test_fused_dq_run_to_run():
    """The order of the fp32 adds changes between runs; the result does not move by more than that."""
    q, k, v, dout = make(2, 4, 4, 1024, 1024, 64, torch.float16, seed=5)
    _, _, first = backward_both(q, k, v, dout, 0.125, 1)
    _, _, second = backward_both(q, k, v, dout, 0.125, 1)
    assert oracle.rel_l2(second[0], first[0]) < 1e-3
    assert torch.equal(first[1], second[1]) and torch.equal(first[2], second[2])


@pytest.mark.parametrize("dim", [64, 128])
def test_autograd_backward_modes(dim):
    """``set_backward``: "fused" and "split" give the same gradients to within the order of fp32 additions,
    "auto" is one of the two, and "split" repeats bit for bit."""
    from kohakufa_b200 import set_backward

    q, k, v, dout = make(1, 2, 2, 640, 640, dim, torch.bfloat16, seed=8, std=0.5)

    def grads():
        leaves = [t.detach().clone().requires_grad_() for t in (q, k, v)]
        attention(*leaves, causal=True).backward(dout)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        return [t.grad for t in leaves]

    got = {}
    try:
        for mode in ("fused", "split", "auto"):
            set_backward(mode)
            got[mode] = grads()
        set_backward("split")
        again = grads()
    finally:
        set_backward("auto")
    for a, b in zip(got["fused"], got["split"]):
        assert oracle.rel_l2(a, b) < 1e-3
    for a, b in zip(got["auto"], got["split"]):
        assert oracle.rel_l2(a, b) < 1e-3
    assert all(torch.equal(a, b) for a, b in zip(again, got["split"]))
