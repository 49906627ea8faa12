"""Forward + backward for callers whose tensors live in HOST memory.

``attention_fwd_bwd_host`` takes pinned host q, k, v, dout and returns pinned host out, dq, dk, dv.
The problem is cut into units of (a few batch entries) x (a group of heads) that flow through three
CUDA streams — host-to-device copies, the attention kernels, device-to-host copies — so the two PCIe
directions and the GPU work overlap instead of running one after the other (at the benchmark's C3
shape the copies are 1.07 GB each way per step and dominate the end-to-end time: what is left outside
the copies is the first unit's way in and the last unit's way out, so units are kept small, about
sixteen per call). A unit of a head group is a strided piece of ``[B, S, H, D]`` storage: it moves
with ONE pitched copy per tensor (``kfa_copy_rows``). Every buffer belongs to a reusable
``HostPipeline``; the kernels are called through the C ABI on preallocated buffers, so a step
allocates nothing.
The reference has no such entry point: its callers hold CUDA tensors (this is plumbing around the
same kernels, for the end-to-end measurement and for hosts that stage data themselves).
"""

import ctypes

import torch

from kohakufa_b200 import _lib
from kohakufa_b200.op import _check, use_fused_backward


def _is_bshd(t: torch.Tensor) -> bool:
    """``[B, H, S, D]`` view of dense ``[B, S, H, D]`` storage."""
    return t.dim() == 4 and t.transpose(1, 2).is_contiguous()


class HostPipeline:
    """Streams plus every device and host buffer for one problem shape: after construction a call
    allocates nothing (two sets of device inputs, results and scratch, used alternately).

    ``slices``: how many units to cut the problem into (default: about 16). Units are whole batch entries
    when there are enough of them; otherwise each batch entry is also cut into groups of K / V heads
    (with the query heads they serve), which needs ``[B, S, H, D]`` host storage."""

    def __init__(self, q, k, v, device, slices=None):
        if not all(t.is_pinned() for t in (q, k, v)):
            raise ValueError("attention_fwd_bwd_host: q, k, v, dout must be pinned host tensors")
        self.device = torch.device(device)
        self.lib = _lib.load()
        batch, heads, seq_q, dim = q.shape
        kv_heads, seq_k = k.shape[1], k.shape[2]
        self.group = heads // kv_heads
        want = slices or 16
        # units: (first batch entry, batch entries, first K / V head, K / V heads)
        head_groups = 1
        if want > batch and all(_is_bshd(t) for t in (q, k, v)):
            head_groups = max(d for d in range(1, kv_heads + 1) if kv_heads % d == 0 and batch * d <= max(want, batch))
        per_unit_batch = max(1, batch // want) if head_groups == 1 else 1
        hk = kv_heads // head_groups
        self.units = [
            (b0, min(per_unit_batch, batch - b0), g * hk, hk)
            for b0 in range(0, batch, per_unit_batch)
            for g in range(head_groups)
        ]
        self.strided = head_groups > 1
        nb = max(u[1] for u in self.units)
        with torch.cuda.device(self.device):
            self.h2d, self.compute, self.d2h = (torch.cuda.Stream() for _ in range(3))
            self.status = _lib.status_word(self.device)

        def dev_buf(n_heads, seq, dtype):  # [nb, S, h, D] storage viewed [nb, h, S, D]
            return torch.empty(nb, seq, n_heads, dim, dtype=dtype, device=self.device).transpose(1, 2)

        def host_like(t):
            return torch.empty(t.shape[0], t.shape[2], t.shape[1], t.shape[3], dtype=t.dtype).pin_memory().transpose(1, 2)

        hq = hk * self.group
        self.inputs = [[dev_buf(hq, seq_q, q.dtype), dev_buf(hk, seq_k, q.dtype), dev_buf(hk, seq_k, q.dtype),
                        dev_buf(hq, seq_q, q.dtype)] for _ in range(2)]  # q, k, v, dout  # fmt: skip
        self.results = [[dev_buf(hq, seq_q, q.dtype), dev_buf(hq, seq_q, q.dtype), dev_buf(hk, seq_k, q.dtype),
                         dev_buf(hk, seq_k, q.dtype)] for _ in range(2)]  # out, dq, dk, dv  # fmt: skip
        self.lse = [torch.empty(nb, hq, 2, seq_q, dtype=torch.float32, device=self.device) for _ in range(2)]
        stats_floats = self.lib.kfa_bwd_stats_bytes(nb, hq, seq_q) // 4
        self.stats = [torch.empty(stats_floats, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.fused = use_fused_backward(dim, nb * hq)
        if self.fused:
            acc_floats = self.lib.kfa_bwd_dq_acc_bytes(nb, hq, seq_q, dim) // 4
            self.dq_acc = [torch.empty(acc_floats, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.outputs = [host_like(q), host_like(q), host_like(k), host_like(v)]  # out, dq, dk, dv
        _check(*self.inputs[0][:3])

    def _attention(self, buf, n, scale, block):
        """Forward + backward of one unit on the current stream through the C entry points."""
        q, k, v, dout = (_lib.tensor4(t[:n]) for t in self.inputs[buf])
        out, dq, dk, dv = (_lib.tensor4(t[:n]) for t in self.results[buf])
        dtype = _lib.dtype_code(self.inputs[buf][0].dtype)
        stream = _lib.stream_ptr(self.device)
        ref = ctypes.byref
        with torch.cuda.device(self.device):
            _lib.check(self.lib.kfa_fwd(ref(q), ref(k), ref(v), ref(out), self.lse[buf].data_ptr(), scale, block, dtype,
                                        self.status.data_ptr(), stream))
            if self.fused:
                _lib.check(self.lib.kfa_bwd_fused(ref(q), ref(k), ref(v), ref(out), ref(dout), self.lse[buf].data_ptr(),
                                                  self.stats[buf].data_ptr(), self.dq_acc[buf].data_ptr(), ref(dq),
                                                  ref(dk), ref(dv), scale, block, dtype, self.status.data_ptr(), stream))
            else:
                _lib.check(self.lib.kfa_bwd(ref(q), ref(k), ref(v), ref(out), ref(dout), self.lse[buf].data_ptr(),
                                            self.stats[buf].data_ptr(), ref(dq), ref(dk), ref(dv), scale, block, dtype,
                                            self.status.data_ptr(), stream))

    def _move(self, dev, host, unit, query_side, to_device):
        """One unit of ``host`` ([B, H, S, D] view) to / from the device buffer ``dev`` on the current stream."""
        b0, n, k0, hk = unit
        h0, nh = (k0 * self.group, hk * self.group) if query_side else (k0, hk)
        piece = host[b0 : b0 + n, h0 : h0 + nh]
        if not self.strided:
            (dev[:n].copy_ if to_device else piece.copy_)(piece if to_device else dev[:n], non_blocking=True)
            return
        # [n, S, nh, D] rows of nh * D elements out of rows of H * D: one pitched copy
        seq, dim, heads = host.shape[2], host.shape[3], host.shape[1]
        row_bytes, pitch = nh * dim * host.element_size(), heads * dim * host.element_size()
        args = (dev.data_ptr(), row_bytes, piece.data_ptr(), pitch) if to_device else (piece.data_ptr(), pitch, dev.data_ptr(), row_bytes)
        assert n == 1 or host.stride(0) == seq * heads * dim  # consecutive batch entries continue the row sequence
        _lib.check(self.lib.kfa_copy_rows(*args, row_bytes, n * seq, int(to_device), _lib.stream_ptr(self.device)))

    def run(self, q, k, v, dout, scale, block):
        cur = torch.cuda.current_stream(self.device)
        for s in (self.h2d, self.compute, self.d2h):
            s.wait_stream(cur)
        done = [None, None]  # the kernels have finished with input set i
        copied = [None, None]  # result set i has left the device
        for idx, unit in enumerate(self.units):
            buf = idx % 2
            n = unit[1]
            with torch.cuda.stream(self.h2d):
                if done[buf] is not None:
                    self.h2d.wait_event(done[buf])
                for d, h, qs in zip(self.inputs[buf], (q, k, v, dout), (True, False, False, True)):
                    self._move(d, h, unit, qs, True)
                ready = torch.cuda.Event()
                ready.record(self.h2d)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(ready)
                if copied[buf] is not None:
                    self.compute.wait_event(copied[buf])
                self._attention(buf, n, scale, block)
                done[buf] = torch.cuda.Event()
                done[buf].record(self.compute)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(done[buf])
                for h, d, qs in zip(self.outputs, self.results[buf], (True, True, False, False)):
                    self._move(d, h, unit, qs, False)
                copied[buf] = torch.cuda.Event()
                copied[buf].record(self.d2h)
        for s in (self.h2d, self.compute, self.d2h):
            cur.wait_stream(s)
        return tuple(self.outputs)


def attention_fwd_bwd_host(q, k, v, dout, *, causal=False, block_causal=0, scale=None, device="cuda", slices=None,
                           pipeline=None):
    """out, dq, dk, dv (pinned host tensors) of ``attention(q, k, v, ...)`` and its backward for ``dout``.
    All four inputs: pinned host ``[B, H, S, D]`` views with a contiguous last dim (e.g. ``[B, S, H, D]``
    storage), fp16 or bf16, head dim a multiple of 16 up to 128. ``pipeline``: a ``HostPipeline`` to reuse buffers and
    streams across calls. The returned host tensors are valid once the current stream has caught up
    (``torch.cuda.current_stream().synchronize()``)."""
    if causal and block_causal not in (0, 1):
        raise ValueError("causal is block_causal=1: give one of them")
    block = 1 if causal else int(block_causal)
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    pipe = pipeline or HostPipeline(q, k, v, device, slices)
    return pipe.run(q, k, v, dout, scale, block)
