"""Context-parallel causal attention: one sequence spread over the N GPUs of a node, K / V passed
around a ring (NCCL send / recv over NVLink), overlapped with the attention kernels.

The reference is single-GPU; this is the multi-GPU piece for sequences that do not fit (or are too
slow on) one GPU, e.g. B=1, H=32, S=131072, D=128. Layout and schedule:

* zig-zag sharding: the sequence is cut into 2N chunks of C rows; rank r owns chunks r and 2N-1-r,
  stored one after the other (local length 2C, local order = global order), which balances the
  causal work;
* step 0 is ordinary causal attention on the local 2C rows; at step t > 0 rank r holds the K / V of
  rank src = (r - t) mod N and runs ONE dense call over half the area: all local queries against the
  first chunk of the visitor (src < r), or the second local chunk against both visiting chunks
  (src > r); every other (query chunk, key chunk) pair is hidden and never launched;
* forward: each step merges its partial result into an fp32 carry (unnormalised O with m and l per
  row, two numbers, never a fused lse); one finalize pass normalises and rounds;
* backward: fp32 dQ accumulates at home; the fp32 dK / dV partials travel with their K / V and come
  home after N hops; everything is rounded to 16 bits once.

Remote data always lands in a local buffer first (double-buffered) and the kernels read it with their
ordinary local TMA loads. ``ring_attention`` is the autograd entry point; ``emulate_ring`` runs all N
ranks of the same schedule in lockstep in one process (tests on a single GPU).
"""

import ctypes

import os

import torch
import torch.distributed as dist

from kohakufa_b200 import _lib


def zigzag_shard(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows of rank ``rank`` (chunks rank and 2*world-1-rank) of a full ``[B, H, S, D]`` tensor, as a
    ``[B, H, 2C, D]`` view of fresh ``[B, 2C, H, D]`` storage."""
    seq = x.shape[2]
    assert seq % (2 * world) == 0
    c = seq // (2 * world)
    a, b = rank, 2 * world - 1 - rank
    rows = torch.cat([x[:, :, a * c : (a + 1) * c], x[:, :, b * c : (b + 1) * c]], dim=2)
    return rows.transpose(1, 2).contiguous().transpose(1, 2)


def zigzag_unshard(parts: list) -> torch.Tensor:
    """Inverse of ``zigzag_shard`` over the list of all ranks' tensors."""
    world = len(parts)
    c = parts[0].shape[2] // 2
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        chunks[r] = p[:, :, :c]
        chunks[2 * world - 1 - r] = p[:, :, c:]
    return torch.cat(chunks, dim=2)


def step_plan(rank: int, world: int, t: int, c: int):
    """(block, (q0, q1), (k0, k1)) of ring step ``t`` on ``rank``: the mask of the one kernel call
    (1 causal, 0 dense) and the local query rows / visiting key rows it covers."""
    src = (rank - t) % world
    if t == 0:
        return 1, (0, 2 * c), (0, 2 * c)
    if src < rank:
        return 0, (0, 2 * c), (0, c)
    return 0, (c, 2 * c), (0, 2 * c)


def _t4(t):
    return ctypes.byref(_lib.tensor4(t))


def _check_local(q, k, v):
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError("ring attention: q, k, v must be [B, H, 2C, D] of one shape")
    if q.shape[-1] not in (64, 128):
        raise ValueError("ring attention: head_dim 64 or 128")
    if q.shape[2] % 256:
        raise ValueError("ring attention: the local length must be a multiple of 256 (chunks of whole tiles)")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("ring attention: fp16 or bf16")


class _Rank:
    """Per-rank buffers and the kernel calls of one ring step (shared by the distributed driver and
    the single-process emulation)."""

    def __init__(self, rank, world, q, scale):
        self.rank, self.world = rank, world
        self.lib = _lib.load()
        self.b, self.h, self.s, self.d = q.shape
        self.c = self.s // 2
        self.scale = float(scale)
        self.code = _lib.dtype_code(q.dtype)
        self.dev = q.device
        self.word = _lib.status_word(q.device).data_ptr()

    def _stream(self):
        return _lib.stream_ptr(self.dev)

    # ---- forward ----
    def fwd_begin(self, q):
        self.o_acc = torch.empty(self.b, self.h, self.s, self.d, dtype=torch.float32, device=self.dev)
        self.ml = torch.empty(self.b, self.h, 2, self.s, dtype=torch.float32, device=self.dev)

    def fwd_step(self, t, q, k_vis, v_vis):
        block, (q0, q1), (k0, k1) = step_plan(self.rank, self.world, t, self.c)
        acc = _lib.acc32(self.o_acc, row0=q0)
        with torch.cuda.device(self.dev):
            _lib.check(
                self.lib.kfa_cp_fwd_step(
                    _t4(q[:, :, q0:q1]), _t4(k_vis[:, :, k0:k1]), _t4(v_vis[:, :, k0:k1]), ctypes.byref(acc),
                    self.ml.data_ptr() + 4 * q0, 2 * self.s, self.s, int(t > 0), self.scale, block, self.code,
                    self.word, self._stream(),
                )
            )

    def fwd_end(self, q):
        out = q.new_empty(self.b, self.s, self.h, self.d).transpose(1, 2)
        lse = q.new_empty(self.b, self.h, 2, self.s, dtype=torch.float32)
        acc = _lib.acc32(self.o_acc)
        with torch.cuda.device(self.dev):
            _lib.check(
                self.lib.kfa_cp_fwd_finalize(ctypes.byref(acc), self.ml.data_ptr(), 2 * self.s, self.s, _t4(out),
                                             lse.data_ptr(), self.code, self._stream())
            )
        del self.o_acc, self.ml
        return out, lse

    # ---- backward ----
    def bwd_begin(self, out, dout, lse):
        self.stats = out.new_empty(self.lib.kfa_bwd_stats_bytes(self.b, self.h, self.s) // 4, dtype=torch.float32)
        self.stats_sh = (self.s // 128) * 384
        self.dq_acc = torch.empty(self.b, self.h, self.s, self.d, dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            _lib.check(self.lib.kfa_bwd_prepare(_t4(out), _t4(dout), lse.data_ptr(), self.stats.data_ptr(), self.code,
                                                self._stream()))

    def bwd_dq_step(self, t, q, dout, k_vis, v_vis):
        block, (q0, q1), (k0, k1) = step_plan(self.rank, self.world, t, self.c)
        acc = _lib.acc32(self.dq_acc, row0=q0)
        with torch.cuda.device(self.dev):
            _lib.check(
                self.lib.kfa_cp_bwd_dq_step(
                    _t4(q[:, :, q0:q1]), _t4(k_vis[:, :, k0:k1]), _t4(v_vis[:, :, k0:k1]), _t4(dout[:, :, q0:q1]),
                    self.stats.data_ptr() + 4 * (q0 // 128) * 384, self.stats_sh, ctypes.byref(acc), int(t > 0),
                    self.scale, block, self.code, self.word, self._stream(),
                )
            )

    def bwd_dkdv_step(self, t, q, dout, k_vis, v_vis, dkv_acc):
        """``dkv_acc``: fp32 [2, B, H, 2C, D], the accumulator that travels with the visiting K / V."""
        block, (q0, q1), (k0, k1) = step_plan(self.rank, self.world, t, self.c)
        dk = _lib.acc32(dkv_acc[0], row0=k0)
        dv = _lib.acc32(dkv_acc[1], row0=k0)
        with torch.cuda.device(self.dev):
            _lib.check(
                self.lib.kfa_cp_bwd_dkdv_step(
                    _t4(q[:, :, q0:q1]), _t4(k_vis[:, :, k0:k1]), _t4(v_vis[:, :, k0:k1]), _t4(dout[:, :, q0:q1]),
                    self.stats.data_ptr() + 4 * (q0 // 128) * 384, self.stats_sh, ctypes.byref(dk), ctypes.byref(dv),
                    int(t > 0), self.scale, block, self.code, self.word, self._stream(),
                )
            )

    def grad_end(self, acc, like):
        grad = like.new_empty(self.b, self.s, self.h, self.d).transpose(1, 2)
        a = _lib.acc32(acc)
        with torch.cuda.device(self.dev):
            _lib.check(self.lib.kfa_cp_grad_finalize(ctypes.byref(a), _t4(grad), self.code, self._stream()))
        return grad


# --------------------------------------------------------------------------------------
# Single-process emulation: all N ranks of the schedule in lockstep on one GPU
# --------------------------------------------------------------------------------------
def emulate_ring(qs, ks, vs, douts, scale=None):
    """Runs the ring schedule for ``world = len(qs)`` ranks whose shards all live on one GPU; "sending"
    is a rotation of the list. Returns per-rank lists (outs, lses, dqs, dks, dvs). The kernel calls,
    buffers and step plans are exactly those of the distributed driver."""
    world = len(qs)
    for q, k, v in zip(qs, ks, vs):
        _check_local(q, k, v)
    scale = qs[0].shape[-1] ** -0.5 if scale is None else scale
    ranks = [_Rank(r, world, qs[r], scale) for r in range(world)]
    # forward
    for r in range(world):
        ranks[r].fwd_begin(qs[r])
    for t in range(world):
        for r in range(world):
            src = (r - t) % world
            ranks[r].fwd_step(t, qs[r], ks[src], vs[src])
    outs, lses = zip(*(ranks[r].fwd_end(qs[r]) for r in range(world)))
    # backward
    for r in range(world):
        ranks[r].bwd_begin(outs[r], douts[r], lses[r])
    dkv = [torch.empty(2, *qs[r].shape, dtype=torch.float32, device=qs[r].device) for r in range(world)]  # by owner
    for t in range(world):
        for r in range(world):
            src = (r - t) % world
            ranks[r].bwd_dq_step(t, qs[r], douts[r], ks[src], vs[src])
            ranks[r].bwd_dkdv_step(t, qs[r], douts[r], ks[src], vs[src], dkv[src])
    dqs = [ranks[r].grad_end(ranks[r].dq_acc, qs[r]) for r in range(world)]
    dks = [ranks[r].grad_end(dkv[r][0], ks[r]) for r in range(world)]
    dvs = [ranks[r].grad_end(dkv[r][1], vs[r]) for r in range(world)]
    return list(outs), list(lses), dqs, dks, dvs


# --------------------------------------------------------------------------------------
# Distributed driver (one process per GPU, torch.distributed / NCCL)
# --------------------------------------------------------------------------------------
def nccl_options():
    """Process-group options for the ring: NCCL's kernels on a HIGH-PRIORITY stream. An attention CTA takes
    nearly all of an SM's shared memory, so a send / receive CTA can only start on an SM that an attention
    CTA has just left; at the default priority the block scheduler hands that SM to the next attention CTA of
    the running grid, the transfer of step t+1 starts when step t's grid has drained, and nothing overlaps
    (measured at 8 GPUs: the compute stream waited 10.2 of 80 ms for transfers; with the priority 1.1 of 73). Pass the result as
    ``pg_options`` to ``init_process_group`` / ``new_group``. (Limiting NCCL's CTAs on top of that — 4, 8,
    16 per message — was measured at 4 GPUs and is no better than NCCL's own choice: 170 / 148 / 145 ms
    against 143.)"""
    opts = dist.ProcessGroupNCCL.Options()
    opts.is_high_priority_stream = True
    return opts


def _shift(tensor_out, tensor_in, group):
    """Starts sending ``tensor_out`` to the next rank and receiving ``tensor_in`` from the previous one;
    returns the requests (wait on them before touching ``tensor_in`` or overwriting ``tensor_out``)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    nxt = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    prv = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    ops = [dist.P2POp(dist.isend, tensor_out, nxt, group), dist.P2POp(dist.irecv, tensor_in, prv, group)]
    return dist.batch_isend_irecv(ops)


def _wait(reqs, trace=None, label="wait"):
    """Makes the compute stream wait for the transfers. With a ``trace`` the stall is bracketed by events:
    the time between them is what the stream spent idle waiting for NCCL."""
    _mark(trace, "begin:" + label)
    for r in reqs:
        r.wait()
    _mark(trace, "end:" + label)


def _mark(trace, label):
    """Appends (label, event recorded now on the current stream) to ``trace`` (a list, or None = off)."""
    if trace is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        trace.append((label, ev))


def trace_summary(trace):
    """Milliseconds per label from a ``trace`` filled by ``ring_forward`` / ``ring_backward``: for every
    ``begin:x`` ... ``end:x`` pair the device time between the two events, summed per ``x`` (the events
    must have completed: synchronise first)."""
    total, open_at = {}, {}
    for label, ev in trace:
        kind, name = label.split(":", 1)
        if kind == "begin":
            open_at[name] = ev
        else:
            total[name] = total.get(name, 0.0) + open_at.pop(name).elapsed_time(ev)
    return total


def _pack_kv(k, v):
    """K and V in one contiguous [2, B, 2C, H, D] buffer (one message per hop)."""
    kv = torch.empty(2, k.shape[0], k.shape[2], k.shape[1], k.shape[3], dtype=k.dtype, device=k.device)
    kv[0].copy_(k.transpose(1, 2))
    kv[1].copy_(v.transpose(1, 2))
    return kv


def _views(kv):
    return kv[0].transpose(1, 2), kv[1].transpose(1, 2)


def ring_forward(q, k, v, scale, group=None, trace=None):
    """out, lse of this rank's queries. The K / V of step t+1 travel while step t computes.
    ``trace``: a list that receives timing marks (see ``trace_summary``)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    _check_local(q, k, v)
    st = _Rank(rank, world, q, scale)
    st.fwd_begin(q)
    cur = _pack_kv(k, v)
    nxt = torch.empty_like(cur) if world > 1 else None
    for t in range(world):
        reqs = _shift(cur, nxt, group) if t + 1 < world else []
        kc, vc = _views(cur)
        _mark(trace, "begin:fwd kernels")
        st.fwd_step(t, q, kc, vc)
        _mark(trace, "end:fwd kernels")
        if reqs:
            _wait(reqs, trace, "fwd wait for K/V")
            cur, nxt = nxt, cur
    return st.fwd_end(q)


def ring_backward(q, k, v, out, dout, lse, scale, group=None, trace=None):
    """dq, dk, dv of this rank's rows. Per step: the dQ kernel runs while the fp32 dK / dV accumulator
    of the visiting K / V is still arriving from the previous rank, then the dK / dV kernel adds to it
    and it moves on; after N hops it is back at its owner."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    st = _Rank(rank, world, q, scale)
    st.bwd_begin(out, dout, lse)
    cur = _pack_kv(k, v)
    nxt = torch.empty_like(cur) if world > 1 else None
    acc = torch.empty(2, *q.shape, dtype=torch.float32, device=q.device)  # for the K / V held now
    acc_in = torch.empty_like(acc) if world > 1 else None
    acc_reqs = []
    for t in range(world):
        kv_reqs = _shift(cur, nxt, group) if t + 1 < world else []
        kc, vc = _views(cur)
        _mark(trace, "begin:bwd dQ kernel")
        st.bwd_dq_step(t, q, dout, kc, vc)
        _mark(trace, "end:bwd dQ kernel")
        if acc_reqs:  # the accumulator for this step's K / V, sent by the previous rank after its step t-1
            _wait(acc_reqs, trace, "bwd wait for dK/dV accumulator")
            acc, acc_in = acc_in, acc
        _mark(trace, "begin:bwd dK/dV kernel")
        st.bwd_dkdv_step(t, q, dout, kc, vc, acc)
        _mark(trace, "end:bwd dK/dV kernel")
        acc_reqs = _shift(acc, acc_in, group) if world > 1 else []
        if kv_reqs:
            _wait(kv_reqs, trace, "bwd wait for K/V")
            cur, nxt = nxt, cur
    if acc_reqs:  # the last hop brings this rank's own accumulator home
        _wait(acc_reqs, trace, "bwd wait for dK/dV accumulator")
        acc = acc_in
    dq = st.grad_end(st.dq_acc, q)
    dk = st.grad_end(acc[0], k)
    dv = st.grad_end(acc[1], v)
    return dq, dk, dv


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, group):
        out, lse = ring_forward(q, k, v, scale, group)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale, ctx.group = scale, group
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, dlse):
        q, k, v, out, lse = ctx.saved_tensors
        if dout.stride(-1) != 1 or any(s % 8 or s <= 0 for n, s in zip(dout.shape[:-1], dout.stride()[:-1]) if n > 1):
            dout = dout.contiguous()
        dq, dk, dv = ring_backward(q, k, v, out, dout, lse, ctx.scale, ctx.group)
        return dq, dk, dv, None, None


def ring_attention(q, k, v, *, scale=None, group=None):
    """Causal attention over a sequence sharded zig-zag across the ranks of ``group`` (default: the
    world). ``q, k, v``: this rank's ``[B, H, 2C, D]`` rows (``zigzag_shard`` of the full tensors).
    Returns this rank's rows of the output; differentiable."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    out, _ = _RingAttention.apply(q, k, v, scale, group)
    return out
