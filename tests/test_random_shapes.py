"""Seeded random problems against the fp64 oracle: head dim, dtype, lengths, grouped heads, mask mode and
backward implementation drawn together, so that combinations no hand-written case lists get exercised
(reference test strategy: tests/test_attention.py parametrises the same axes one or two at a time)."""

import os
import random

import pytest
import torch

from kohakufa_b200 import _lib, attention, set_backward
from oracle import reference as oracle

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    dim = rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 24, 100])
    dtype = rng.choice([torch.float16, torch.bfloat16])
    kv_heads = rng.choice([1, 2, 3])
    group = rng.choice([1, 1, 2, 4])
    batch = rng.choice([1, 2])
    s_q = rng.choice([1, 7, 64, 127, 128, 129, 200, 255, 256, 257, 300, 383, 500, 641])
    mode = rng.choice(["dense", "causal", "block", "mask"])
    s_kv = s_q if mode in ("causal", "block") and rng.random() < 0.7 else rng.choice([1, 33, 128, 129, 260, 390, 517])
    block = {"dense": 0, "causal": 1, "block": rng.choice([2, 16, 100, 128, 130, 256]), "mask": 0}[mode]
    backward = rng.choice(["auto", "split", "fused"])
    return dim, dtype, batch, kv_heads, group, s_q, s_kv, mode, block, backward


@pytest.mark.parametrize("seed", range(int(os.environ.get("KFA_RANDOM_CASES", "64"))))
def test_random_problem(seed):
    dim, dtype, batch, kv_heads, group, s_q, s_kv, mode, block, backward = draw(seed)
    heads = kv_heads * group
    gen = torch.Generator().manual_seed(1000 + seed)

    def projection(seq, n_heads):
        return torch.randn(batch, seq, n_heads, dim, generator=gen).to(dtype).cuda().transpose(1, 2).requires_grad_()

    q, k, v = projection(s_q, heads), projection(s_kv, kv_heads), projection(s_kv, kv_heads)
    dout = torch.randn(batch, heads, s_q, dim, generator=gen).to(dtype).cuda()
    kwargs, mask = {}, None
    if mode == "causal":
        kwargs["causal"] = True
    elif mode == "block":
        kwargs["block_causal"] = block
    elif mode == "mask":
        mask = (torch.rand(batch, heads, s_q, s_kv, generator=gen) < 0.6).cuda()
        mask[..., 0] = True  # every row sees a key: the comparison below is relative
        kwargs["mask"] = mask
    set_backward(backward)
    try:
        out = attention(q, k, v, **kwargs)
        out.backward(dout)
        torch.cuda.synchronize()
    finally:
        set_backward("auto")
    assert _lib.device_status() == 0
    kk, vv = (t.detach().repeat_interleave(group, dim=1) for t in (k, v))
    want_out, want_dq, dkk, dvv = oracle.attention_fp64(q, kk, vv, dout, dim**-0.5, block=block, mask=mask)
    want_dk = dkk.reshape(batch, kv_heads, group, s_kv, dim).sum(2)
    want_dv = dvv.reshape(batch, kv_heads, group, s_kv, dim).sum(2)
    tol = 5e-3 if dtype == torch.float16 else 2e-2  # relative error against fp64, per dtype
    for name, g, w in zip(("out", "dq", "dk", "dv"), (out, q.grad, k.grad, v.grad), (want_out, want_dq, want_dk, want_dv)):
        assert bool(torch.isfinite(g).all()), (name, draw(seed))
        m = oracle.metrics(g, w)
        if float(w.abs().max()) == 0.0:
            assert m["max_abs_err"] < 1e-4, (name, m, draw(seed))
        else:
            assert m["rel_err"] < tol, (name, m, draw(seed))
