"""``kfa_bwd_static_scratch``: the backward for hosts that cannot give the library a scratch buffer
(a binding with no device allocator of its own, a loop that must stay clear of cudaMalloc). It keeps
the per-row statistics in a fixed buffer inside the library instead of the caller's ``stats``.

Checked here through the C ABI: two calls in a row must reproduce, bit for bit, what ``kfa_bwd`` gives
with a caller-allocated buffer (the kernels are the same and deterministic), also when the second
call is a different, smaller problem that only overwrites part of the shared buffer; and a problem
beyond the stated limit must be refused without touching the GPU. This file sorts last on purpose:
a run that stops at the first failure has then already been through every other test."""

import ctypes

import pytest
import torch

from kohakufa_b200 import _lib
from kohakufa_b200.op import attention_fwd_op

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 8 * 1024 * 1024  # KFA_STATIC_SCRATCH_BYTES in include/kfa.h


def _like(t):
    return t.new_empty(t.shape[0], t.shape[2], t.shape[1], t.shape[3]).transpose(1, 2)


def _problem(batch, heads, seq, dim, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    q, k, v, dout = (
        torch.randn(batch, seq, heads, dim, generator=gen).to(dtype).cuda().transpose(1, 2) for _ in range(4)
    )
    return q, k, v, dout


def _backward_both_ways(q, k, v, dout, block):
    """(dq, dk, dv) from kfa_bwd with a caller buffer, and from kfa_bwd_static_scratch."""
    lib = _lib.load()
    scale = q.shape[-1] ** -0.5
    out, lse = attention_fwd_op(q, k, v, scale, block)
    code = _lib.dtype_code(q.dtype)
    word = _lib.status_word(q.device).data_ptr()
    stream = _lib.stream_ptr(q.device)
    t = {n: ctypes.byref(_lib.tensor4(x)) for n, x in dict(q=q, k=k, v=v, out=out, dout=dout).items()}

    want = [_like(q), _like(k), _like(v)]
    stats = q.new_empty(lib.kfa_bwd_stats_bytes(q.shape[0], q.shape[1], q.shape[2]) // 4, dtype=torch.float32)
    _lib.check(
        lib.kfa_bwd(t["q"], t["k"], t["v"], t["out"], t["dout"], lse.data_ptr(), stats.data_ptr(),
                    *(ctypes.byref(_lib.tensor4(x)) for x in want), scale, block, code, word, stream)
    )
    got = [_like(q), _like(k), _like(v)]
    for x in got:
        x.fill_(float("nan"))  # the entry point has to write every element itself
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]  # bytes the driver can still hand out on this device
    _lib.check(
        lib.kfa_bwd_static_scratch(t["q"], t["k"], t["v"], t["out"], t["dout"], lse.data_ptr(),
                                   *(ctypes.byref(_lib.tensor4(x)) for x in got), scale, block, code, word, stream)
    )
    torch.cuda.synchronize()
    # "allocates nothing", observed: the device's free memory is the same after the call as before it
    # (torch's caching allocator is not involved either: no torch call sits between the two readings)
    assert torch.cuda.mem_get_info()[0] == free_before
    assert _lib.device_status() == 0
    return want, got


def test_static_scratch_backward_matches_twice_in_a_row():
    # first call: 2 x 3 heads, 700 rows -> 36 statistic tiles
    q, k, v, dout = _problem(2, 3, 700, 64, torch.float16, seed=21)
    want, got = _backward_both_ways(q, k, v, dout, block=1)
    for name, w, g in zip(("dq", "dk", "dv"), want, got):
        assert torch.equal(w, g), name
    # second call right after: another dtype, head dim and mask, fewer tiles, so most of the shared
    # buffer still holds the first call's statistics
    q, k, v, dout = _problem(1, 2, 389, 128, torch.bfloat16, seed=22)
    want, got = _backward_both_ways(q, k, v, dout, block=0)
    for name, w, g in zip(("dq", "dk", "dv"), want, got):
        assert torch.equal(w, g), name
        assert bool(torch.isfinite(g).all()), name


def test_static_scratch_refuses_problems_beyond_its_limit():
    lib = _lib.load()
    # 44 x 128 heads-tiles: ceil(129 / 128) = 2 tiles per head -> 5632 * 2 > 5461 tiles
    batch, heads, seq = 44, 128, 129
    assert lib.kfa_bwd_stats_bytes(batch, heads, seq) > STATIC_SCRATCH_BYTES
    x = torch.zeros(1, dtype=torch.float16, device="cuda")
    d = _lib.KfaTensor4()
    d.ptr = x.data_ptr()
    for i, (n, s) in enumerate(zip((batch, heads, seq, 64), (heads * seq * 64, seq * 64, 64, 1))):
        d.shape[i], d.stride[i] = n, s
    ref = ctypes.byref(d)
    rc = lib.kfa_bwd_static_scratch(ref, ref, ref, ref, ref, x.data_ptr(), ref, ref, ref, 0.125, 0, 0,
                                    _lib.status_word(x.device).data_ptr(), None)
    assert rc == -1
    message = lib.kfa_last_error().decode()
    assert "built-in" in message and "kfa_bwd" in message
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
