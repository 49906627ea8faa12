"""GPU parity tests of ``attention_varlen`` (packed variable-length batches): every sequence of the
batch against the fp64 oracle, and bit for bit against ``attention`` on that sequence alone.
Lengths, head counts and tolerances follow the reference's varlen tests (KohakuFA
tests/test_attention.py:271-344)."""

import pytest
import torch

from kohakufa_b200 import _lib, attention, attention_varlen, set_deterministic, varlen_plan
from oracle import reference as oracle

pytestmark = pytest.mark.gpu

TOL = 5e-3
BF16_TOL = 2e-2


def packed(len_q, len_k, heads, kv_heads, dtype=torch.float16, seed=4, dim=64):
    """Packed q [Tq, H, D], k / v [Tk, Hkv, D], dout and the two cu_seqlens (generated on the CPU)."""
    gen = torch.Generator().manual_seed(seed)

    def cu(lengths):
        return torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device="cuda")

    def make(total, h):
        return torch.randn(total, h, dim, generator=gen).to(dtype).cuda().requires_grad_()

    q = make(sum(len_q), heads)
    k, v = make(sum(len_k), kv_heads), make(sum(len_k), kv_heads)
    dout = torch.randn(sum(len_q), heads, dim, generator=gen).to(dtype).cuda()
    return q, k, v, dout, cu(len_q), cu(len_k)


def as4(t, s, e):
    return t[s:e].unsqueeze(0).transpose(1, 2)


def check_varlen(len_q, len_k, heads, kv_heads, block, dtype=torch.float16, tol=TOL, dim=64, **kwargs):
    q, k, v, dout, cu_q, cu_k = packed(len_q, len_k, heads, kv_heads, dtype, dim=dim)
    out = attention_varlen(q, k, v, cu_q, cu_k, block_causal=block, **kwargs)
    out.backward(dout)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    group = heads // kv_heads
    for b in range(len(len_q)):
        sq, eq = int(cu_q[b]), int(cu_q[b + 1])
        sk, ek = int(cu_k[b]), int(cu_k[b + 1])
        if eq == sq:
            continue
        q1, k1, v1 = as4(q.detach(), sq, eq), as4(k.detach(), sk, ek), as4(v.detach(), sk, ek)
        d1 = as4(dout, sq, eq)
        got = (as4(out, sq, eq), as4(q.grad, sq, eq), as4(k.grad, sk, ek), as4(v.grad, sk, ek))
        # fp64 oracle on this sequence alone
        kk, vv = (t.repeat_interleave(group, dim=1) for t in (k1, v1))
        w_out, w_dq, w_dkk, w_dvv = oracle.attention_fp64(q1, kk, vv, d1, dim**-0.5, block=block)
        w_dk = w_dkk.reshape(1, kv_heads, group, ek - sk, dim).sum(2)
        w_dv = w_dvv.reshape(1, kv_heads, group, ek - sk, dim).sum(2)
        for name, g, w in zip(("out", "dq", "dk", "dv"), got, (w_out, w_dq, w_dk, w_dv)):
            assert bool(torch.isfinite(g).all()), (b, name)
            m = oracle.metrics(g, w)
            if float(w.abs().max()) == 0.0:
                assert m["max_abs_err"] < 1e-4, (b, name, m)
            else:
                assert m["rel_err"] < tol, (b, name, m)
        # the same kernels on the sequence as a batch of one: identical bits (tiles are numbered from
        # the sequence's first row, and what a tile reads of its neighbours is masked)
        qa, ka, va = (t.clone().requires_grad_() for t in (q1, k1, v1))
        set_deterministic(True)  # packed batches run the split backward kernels: compare like with like
        try:
            alone = attention(qa, ka, va, block_causal=block)
            alone.backward(d1)
        finally:
            set_deterministic(False)
        for name, g, w in zip(("out", "dq", "dk", "dv"), got, (alone, qa.grad, ka.grad, va.grad)):
            assert torch.equal(g, w), (b, name)


@pytest.mark.parametrize(
    "lengths,heads,kv_heads,block",
    [
        ([5, 300, 129, 1000, 256], 4, 4, 0),
        ([1, 77, 512, 3, 1300], 8, 2, 1),
        ([600, 257, 24], 3, 3, 24),
        ([128, 256, 384], 2, 1, 0),
    ],
    ids=str,
)
def test_varlen(lengths, heads, kv_heads, block):
    check_varlen(lengths, lengths, heads, kv_heads, block)


def test_varlen_bf16():
    check_varlen([300, 129, 700], [300, 129, 700], 4, 2, 1, dtype=torch.bfloat16, tol=BF16_TOL)


@pytest.mark.parametrize("dim", [32, 80])
def test_varlen_native_head_dims(dim):
    check_varlen([700, 130, 256], [700, 130, 256], 4, 2, 1, dtype=torch.bfloat16, tol=BF16_TOL, dim=dim)


def test_varlen_dim128_bf16():
    check_varlen([700, 130, 256], [700, 130, 256], 2, 2, 1, dtype=torch.bfloat16, tol=BF16_TOL, dim=128)


@pytest.mark.parametrize("block", [0, 1, 100])
def test_varlen_different_query_and_key_lengths(block):
    """cu_seqlens_q != cu_seqlens_k (cross attention per sequence), with an empty sequence in the batch."""
    check_varlen([200, 0, 64, 513], [333, 0, 700, 129], 2, 2, block)


def test_varlen_keys_without_queries_get_zero_gradients():
    q, k, v, dout, cu_q, cu_k = packed([0, 150], [200, 150], 2, 2)
    attention_varlen(q, k, v, cu_q, cu_k).backward(dout)
    assert float(k.grad[:200].abs().max()) == 0.0 and float(v.grad[:200].abs().max()) == 0.0
    assert float(k.grad[200:].abs().max()) > 0.0


def test_varlen_head_dim_padding_and_center_keys():
    q, k, v, dout, cu, _ = packed([300, 129, 50], [300, 129, 50], 2, 2, dim=40)
    out = attention_varlen(q, k, v, cu, cu, causal=True, center_keys=True)
    out.backward(dout)
    assert out.shape == q.shape
    for b in range(3):
        s, e = int(cu[b]), int(cu[b + 1])
        q1, k1, v1 = (as4(t.detach(), s, e) for t in (q, k, v))
        want = oracle.attention_fp64(q1, k1, v1, as4(dout, s, e), 40**-0.5, block=1)
        got = (as4(out, s, e), as4(q.grad, s, e), as4(k.grad, s, e), as4(v.grad, s, e))
        for name, g, w in zip(("out", "dq", "dk", "dv"), got, want):
            assert oracle.metrics(g, w)["rel_err"] < TOL, (b, name)


def test_varlen_cuda_graph():
    """With a plan built beforehand the call makes no host synchronisation: capturable
    (reference test: tests/test_attention.py:323-344)."""
    q, k, v, dout, cu, _ = packed([300, 129, 700], [300, 129, 700], 4, 4)
    plan = varlen_plan(cu, cu, 4, 4, 1)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            attention_varlen(q, k, v, cu, cu, causal=True, plan=plan).backward(dout)
        for t in (q, k, v):
            t.grad = None
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = attention_varlen(q, k, v, cu, cu, causal=True, plan=plan)
            out.backward(dout)
    torch.cuda.current_stream().wait_stream(stream)
    graph.replay()
    torch.cuda.synchronize()
    eager = attention_varlen(*(t.detach() for t in (q, k, v)), cu, cu, causal=True)
    assert torch.equal(out, eager)
    assert bool(torch.isfinite(q.grad).all()) and float(q.grad.abs().max()) > 0


def test_varlen_argument_errors():
    q, k, v, _, cu, _ = packed([100, 50], [100, 50], 2, 2)
    with pytest.raises(ValueError):
        attention_varlen(q, k, v, cu, cu, causal=True, block_causal=5)
    with pytest.raises(ValueError):  # a plan for another number of sequences
        attention_varlen(q, k, v, cu, cu, plan=(3, 100, 100))
    with pytest.raises(ValueError):  # queries without keys
        varlen_plan(cu, torch.tensor([0, 150, 150], dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError):
        attention_varlen(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), cu, cu)


def test_sequence_without_keys_through_a_user_plan():
    """``varlen_plan`` refuses a sequence that has queries but no keys; a caller that hands in its own plan
    skips that check. Such rows then see nothing: output 0 and zero gradients (what the reference documents
    for a query row without a visible key), never uninitialised memory."""
    len_q, len_k = [70, 40, 130], [90, 0, 130]
    q, k, v, dout, cu_q, cu_k = packed(len_q, len_k, 2, 2)
    plan = (3, 130, 130)  # (sequences, longest query length, longest key length) written by hand
    out = attention_varlen(q, k, v, cu_q, cu_k, causal=True, plan=plan)
    out.backward(dout)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert float(out[70:110].abs().max()) == 0.0 and float(q.grad[70:110].abs().max()) == 0.0
    for b in (0, 2):  # the other sequences are unaffected
        sq, eq, sk, ek = int(cu_q[b]), int(cu_q[b + 1]), int(cu_k[b]), int(cu_k[b + 1])
        want = oracle.attention_fp64(as4(q.detach(), sq, eq), as4(k.detach(), sk, ek), as4(v.detach(), sk, ek),
                                     as4(dout, sq, eq), 64**-0.5, block=1)  # fmt: skip
        got = (as4(out, sq, eq), as4(q.grad, sq, eq), as4(k.grad, sk, ek), as4(v.grad, sk, ek))
        for g, w in zip(got, want):
            assert oracle.metrics(g, w)["rel_err"] < TOL
