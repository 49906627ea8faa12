"""GPU tests at the benchmark configurations' FULL sizes (C3: causal bf16 B4 H32 S8192 D128; C4: block-causal
fp16 P=256 B8 H16 S4096 D64 and dense S=4100), where an fp64 S x S oracle per head is too slow to run
for every head: size-independent identities of attention that any correct kernel satisfies, over all
heads and rows, plus the fp64 oracle on a few (batch, head) slices.

  * softmax rows sum to 1:   V = 1  =>  out = 1;  sum over keys of dV = sum over queries of dO
  * rows of dS sum to 0:     sum over keys of dK = 0
  * a row that sees one key (causal row 0) copies it:  out[0] = v[0], dq[0] ~ 0
  * the same call twice gives the same bits
"""

import pytest
import torch

from kohakufa_b200 import _lib, attention, workloads
from oracle import reference as oracle

pytestmark = pytest.mark.gpu


def run(cfg, q, k, v, dout):
    q, k, v = (t.detach().requires_grad_() for t in (q, k, v))
    kwargs = {"causal": True} if cfg.block == 1 else ({"block_causal": cfg.block} if cfg.block else {})
    out = attention(q, k, v, **kwargs)
    out.backward(dout)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return out, q.grad, k.grad, v.grad


@pytest.mark.parametrize("name", ["C3", "C4", "C4-dense4100"])
def test_identities_at_full_size(name):
    cfg = workloads.CONFIGS[name]
    q, k, v, dout = (t.cuda() for t in workloads.make_inputs(cfg))
    tol = 2e-2 if cfg.dtype == torch.bfloat16 else 5e-3
    out, dq, dk, dv = run(cfg, q, k, v, dout)
    for t in (out, dq, dk, dv):
        assert bool(torch.isfinite(t).all())
    # sum over keys of dV = sum over queries of dO (rows of P sum to 1), per (batch, head)
    want = dout.double().sum(2)
    assert oracle.metrics(dv.double().sum(2), want)["rel_err"] < tol
    # sum over keys of dK = 0 (rows of dS sum to 0): small against the size of dK's rows
    scale_ref = dk.double().abs().sum(2)
    assert float((dk.double().sum(2).abs() / scale_ref.clamp_min(1e-30)).max()) < tol
    if cfg.block == 1:  # causal: row 0 sees key 0 only
        assert torch.equal(out[:, :, 0], v[:, :, 0])
        assert float(dq[:, :, 0].abs().max()) < 1e-3 * float(dq.abs().max())  # dP - delta cancels to rounding
    # the same bits again (dQ: up to the order of the fused backward's fp32 additions)
    again = run(cfg, q, k, v, dout)
    for a, b in zip((out, dk, dv), (again[0], again[2], again[3])):
        assert torch.equal(a, b)
    assert oracle.metrics(again[1], dq.double())["rel_err"] < 1e-3
    # V = 1: every output element is 1 up to the rounding of P (the normaliser sums the unrounded P)
    ones = torch.ones_like(v)
    out1 = run(cfg, q, k, ones, dout)[0]
    assert float((out1.float() - 1.0).abs().max()) < tol
    del out1, again
    # fp64 oracle on three (batch, head) slices: first, a middle one, last
    b_h = [(0, 0), (cfg.batch // 2, cfg.heads // 2), (cfg.batch - 1, cfg.heads - 1)]
    for b, h in b_h:
        sl = lambda t: t[b : b + 1, h : h + 1]  # noqa: E731
        want = oracle.attention_fp64(sl(q), sl(k), sl(v), sl(dout), cfg.scale, block=cfg.block)
        for nm, g, w in zip(("out", "dq", "dk", "dv"), (out, dq, dk, dv), want):
            assert oracle.metrics(sl(g), w)["rel_err"] < tol, (name, b, h, nm)
        del want
