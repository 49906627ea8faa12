"""CPU oracle for the attention hot path. TEST INFRASTRUCTURE ONLY: nothing in the product
(``kohakufa_b200/``) imports this; only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` do.

A restatement, in explicit formulas, of what the reference checks its kernels against:

* ``visible``            KohakuFA tests/reference.py:6-12   (block-causal visibility, top-left aligned)
* ``attention_fp64``     KohakuFA tests/reference.py:15-34  (fp64 attention; the reference gets the
                         gradients from autograd, this file writes the backward out by hand)
* ``metrics``            KohakuFA tests/reference.py:37-47
* ``floor_grads``        KohakuFA benchmarks/dinov3_backward.py:227-263 (``emulated_grads``): a flash
                         backward in fp64 whose tensor-core operands (P for P.V, O, dS) are rounded to
                         the 16-bit dtype: the error ANY correct 16-bit kernel pays ("the floor"). The
                         three named bugs are kept as negative controls.
* ``rel_l2``             KohakuFA benchmarks/dinov3_backward.py:275-281

Parity is pinned: ``tests/golden/make_golden.py`` ran the reference's own two functions (imported
from the reference checkout) on seeded CPU inputs and stored their outputs in
``tests/golden/*.npz``; ``tests/test_oracle.py`` checks this file against them.
"""

import math

import torch

LOG2E = 1.4426950408889634


def visible(s_q: int, s_kv: int, block: int, device="cpu"):
    """Bool [Sq, Skv], True where key c is visible to query r: ``c // block <= r // block``
    (top-left aligned when Sq != Skv). ``None`` for dense attention (block == 0)."""
    if block == 0:
        return None
    rows = torch.arange(s_q, device=device).div(block, rounding_mode="floor").unsqueeze(1)
    cols = torch.arange(s_kv, device=device).div(block, rounding_mode="floor").unsqueeze(0)
    return cols <= rows


def attention_fp64(q, k, v, dout, scale, block=0, mask=None, groups=1):
    """out, dq, dk, dv in fp64 from the given (already rounded) inputs ``[B, H, S, D]``.

    Forward: S = scale q k^T, hidden entries -inf, P = softmax(S), out = P v.
    Backward, written out: dV = P^T dO; dP = dO v^T; delta = rowsum(dO * out);
    dS = P * (dP - delta); dQ = scale dS k; dK = scale dS^T q.
    ``mask`` (instead of ``block``): bool, broadcastable to the scores, True = visible; a query row
    with no visible key has P = 0: output 0 and no gradient (KohakuFA tests/reference.py:27-31).
    ``groups`` > 1: grouped-query attention, each K / V head serves ``groups`` consecutive query heads
    and its dK / dV sum over them (tests/reference.py:22-24)."""
    q, k, v, dout = (t.detach().to(torch.float64) for t in (q, k, v, dout))
    kv_heads = k.shape[1]
    if groups > 1:
        k, v = (t.repeat_interleave(groups, dim=1) for t in (k, v))
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if mask is None:
        mask = visible(q.shape[-2], k.shape[-2], block, q.device)
    if mask is not None:
        mask = mask.expand_as(s)
        rows = mask.any(-1, keepdim=True)
        s = torch.where(rows, s.masked_fill(~mask, float("-inf")), torch.zeros_like(s))
        p = torch.softmax(s, dim=-1) * rows
    else:
        p = torch.softmax(s, dim=-1)
    out = torch.matmul(p, v)
    dv = torch.matmul(p.transpose(-1, -2), dout)
    dp = torch.matmul(dout, v.transpose(-1, -2))
    delta = (dout * out).sum(-1, keepdim=True)
    ds = p * (dp - delta)
    dq = torch.matmul(ds, k) * scale
    dk = torch.matmul(ds.transpose(-1, -2), q) * scale
    if groups > 1:
        shape = (k.shape[0], kv_heads, groups, k.shape[2], k.shape[3])
        dk, dv = dk.reshape(shape).sum(2), dv.reshape(shape).sum(2)
    return out, dq, dk, dv


def metrics(got, want) -> dict:
    """Error of ``got`` against the fp64 ``want``."""
    g = got.detach().to(torch.float64).flatten()
    w = want.detach().to(torch.float64).flatten()
    diff = g - w
    tiny = 1e-300
    return {
        "cos": float(torch.dot(g, w) / (g.norm() * w.norm()).clamp_min(tiny)),
        "norm_ratio": float(g.norm() / w.norm().clamp_min(tiny)),
        "rel_err": float(diff.norm() / w.norm().clamp_min(tiny)),
        "max_abs_err": float(diff.abs().max()),
        "max_rel_err": float(diff.abs().max() / w.abs().max().clamp_min(tiny)),
    }


def rel_l2(got, ref) -> float:
    return float((got.double() - ref.double()).norm() / ref.double().norm())


def floor_grads(q, k, v, dout, scale, block=0, bugs=frozenset(), scores=None):
    """dq, dk, dv (fp64 tensors) of an emulated flash backward whose only errors are the roundings a
    correct 16-bit tensor-core kernel cannot avoid; ``bugs`` adds "scale*dS", "single lse" and / or
    "scale-shift" (each a known way to lose accuracy at large logits).

    Steps a kernel does in fp32 are rounded to fp32 here; the inputs' dtype is the 16-bit dtype.

    ``scores`` (not in the reference's emulation): the raw fp32 scores q k^T as the accumulating
    hardware produces them. By default they are the exact product rounded once to fp32, which no
    tensor core delivers: it sums the D products in groups with a truncating fp32 adder and lands a
    few units in the last place away. At logits ~1e5 one such unit is ~1% of a neighbouring P, so
    the floor of a kernel whose scores come from the tensor core is the one computed from those
    scores (every such kernel pays it, whatever else it does right)."""
    dtype = q.dtype

    def r16(x):
        return x.to(dtype).to(torch.float64)

    def r32(x):
        return x.to(torch.float32).to(torch.float64)

    qd, kd, vd, dod = (t.detach().to(torch.float64) for t in (q, k, v, dout))
    c = r32(torch.tensor(scale * LOG2E, dtype=torch.float64))
    if scores is None:
        s = r32(torch.matmul(qd, kd.transpose(-1, -2)))  # raw scores, fp32 accumulator
    else:
        s = scores.detach().to(torch.float32).to(torch.float64)
    mask = visible(q.shape[-2], k.shape[-2], block, q.device)
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    m = s.amax(-1, keepdim=True)
    if "scale-shift" in bugs:
        expo = r32(s * c - r32(c * m))
    else:
        expo = r32(r32(s - m) * c)
    p_un = torch.exp2(expo)
    l = p_un.sum(-1, keepdim=True)
    out = r16(torch.matmul(r16(p_un), vd) / l)
    delta = (dod * out).sum(-1, keepdim=True)
    if "single lse" in bugs:
        lse = r32(c * m + torch.log2(l))
        p = torch.exp2(r32(s * c - lse))
    else:
        p = torch.exp2(r32(r32(s - m) * c - torch.log2(l)))
    ds = p * (torch.matmul(dod, vd.transpose(-1, -2)) - delta)
    dv = torch.matmul(r16(p).transpose(-1, -2), dod)
    if "scale*dS" in bugs:
        ds = r16(ds * scale)
        return torch.matmul(ds, kd), torch.matmul(ds.transpose(-1, -2), qd), dv
    ds = r16(ds)
    return torch.matmul(ds, kd) * scale, torch.matmul(ds.transpose(-1, -2), qd) * scale, dv


def attention_flops(batch, heads, s_q, s_kv, dim, block=0, backward=True) -> float:
    """Algorithmic FLOPs, the reference's convention (benchmarks/speed.py:21-26, 93, 108):
    forward = 4 B H Sq Skv D x visible fraction; forward + backward = 3.5 x forward."""
    if block == 0:
        pairs = s_q * s_kv
    else:
        rows = torch.arange(s_q, dtype=torch.int64)
        lim = torch.clamp((rows // block + 1) * block, max=s_kv)
        pairs = int(lim.sum())
    fwd = 4.0 * batch * heads * pairs * dim
    return fwd * (3.5 if backward else 1.0)


def _self_check():  # pragma: no cover - manual sanity run
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(1, 2, 33, 16, generator=g).half() for _ in range(4))
    out, dq, dk, dv = attention_fp64(q, k, v, do, 16**-0.5, block=5)
    fq, fk, fv = floor_grads(q, k, v, do, 16**-0.5, block=5)
    print(rel_l2(fq, dq), rel_l2(fk, dk), rel_l2(fv, dv), math.isfinite(float(out.sum())))


if __name__ == "__main__":
    _self_check()
