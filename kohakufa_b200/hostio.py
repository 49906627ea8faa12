"""Forward + backward for callers whose tensors live in HOST memory.

``attention_fwd_bwd_host`` takes pinned host q, k, v, dout and returns pinned host out, dq, dk, dv.
The batch is cut into slices that flow through three CUDA streams — host-to-device copies, the
attention kernels, device-to-host copies — so the two PCIe directions and the GPU work overlap
instead of running one after the other (at the benchmark's C3 shape the copies are 1.07 GB each way
per step and dominate the end-to-end time). Every buffer belongs to a reusable ``HostPipeline``; the kernels are called through the C ABI on
preallocated slices, so a step allocates nothing.
The reference has no such entry point: its callers hold CUDA tensors (this is plumbing around the
same kernels, for the end-to-end measurement and for hosts that stage data themselves).
"""

import ctypes

import torch

from kohakufa_b200 import _lib
from kohakufa_b200.op import _check, use_fused_backward


class HostPipeline:
    """Streams plus every device and host buffer for one problem shape: after construction a call
    allocates nothing (two sets of device inputs, results and statistics, used alternately)."""

    def __init__(self, q, k, v, device, slices=None):
        if not all(t.is_pinned() for t in (q, k, v)):
            raise ValueError("attention_fwd_bwd_host: q, k, v, dout must be pinned host tensors")
        self.device = torch.device(device)
        self.lib = _lib.load()
        self.batch = q.shape[0]
        self.slices = min(self.batch, slices or self.batch)
        self.bounds = [(i * self.batch // self.slices, (i + 1) * self.batch // self.slices) for i in range(self.slices)]
        n = max(b - a for a, b in self.bounds)
        heads, seq_q = q.shape[1], q.shape[2]
        with torch.cuda.device(self.device):
            self.h2d, self.compute, self.d2h = (torch.cuda.Stream() for _ in range(3))
            self.status = _lib.status_word(self.device)

        def dev_like(t):  # [n, S, H, D] storage viewed [n, H, S, D]
            return torch.empty(n, t.shape[2], t.shape[1], t.shape[3], dtype=t.dtype, device=self.device).transpose(1, 2)

        def host_like(t):
            return torch.empty(t.shape[0], t.shape[2], t.shape[1], t.shape[3], dtype=t.dtype).pin_memory().transpose(1, 2)

        self.inputs = [[dev_like(t) for t in (q, k, v, q)] for _ in range(2)]  # q, k, v, dout
        self.results = [[dev_like(t) for t in (q, q, k, v)] for _ in range(2)]  # out, dq, dk, dv
        stats_floats = self.lib.kfa_bwd_stats_bytes(n, heads, seq_q) // 4
        self.lse = [torch.empty(n, heads, 2, seq_q, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.stats = [torch.empty(stats_floats, dtype=torch.float32, device=self.device) for _ in range(2)]
        acc_floats = self.lib.kfa_bwd_dq_acc_bytes(n, heads, seq_q, q.shape[3]) // 4
        self.dq_acc = [torch.empty(acc_floats, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.outputs = [host_like(q), host_like(q), host_like(k), host_like(v)]  # out, dq, dk, dv
        _check(*self.inputs[0][:3])

    def _attention(self, buf, n, scale, block):
        """Forward + backward of one slice on the current stream through the C entry points."""
        q, k, v, dout = (_lib.tensor4(t[:n]) for t in self.inputs[buf])
        out, dq, dk, dv = (_lib.tensor4(t[:n]) for t in self.results[buf])
        dtype = _lib.dtype_code(self.inputs[buf][0].dtype)
        stream = _lib.stream_ptr(self.device)
        ref = ctypes.byref
        with torch.cuda.device(self.device):
            _lib.check(self.lib.kfa_fwd(ref(q), ref(k), ref(v), ref(out), self.lse[buf].data_ptr(), scale, block, dtype,
                                        self.status.data_ptr(), stream))
            if not use_fused_backward(self.inputs[buf][0].shape[3], n * self.inputs[buf][0].shape[1]):
                _lib.check(self.lib.kfa_bwd(ref(q), ref(k), ref(v), ref(out), ref(dout), self.lse[buf].data_ptr(),
                                            self.stats[buf].data_ptr(), ref(dq), ref(dk), ref(dv), scale, block, dtype,
                                            self.status.data_ptr(), stream))
            else:
                _lib.check(self.lib.kfa_bwd_fused(ref(q), ref(k), ref(v), ref(out), ref(dout), self.lse[buf].data_ptr(),
                                                  self.stats[buf].data_ptr(), self.dq_acc[buf].data_ptr(), ref(dq),
                                                  ref(dk), ref(dv), scale, block, dtype, self.status.data_ptr(), stream))

    def run(self, q, k, v, dout, scale, block):
        cur = torch.cuda.current_stream(self.device)
        for s in (self.h2d, self.compute, self.d2h):
            s.wait_stream(cur)
        done = [None, None]  # the kernels have finished with input set i
        copied = [None, None]  # result set i has left the device
        for idx, (a, b) in enumerate(self.bounds):
            buf = idx % 2
            n = b - a
            with torch.cuda.stream(self.h2d):
                if done[buf] is not None:
                    self.h2d.wait_event(done[buf])
                for d, h in zip(self.inputs[buf], (q, k, v, dout)):
                    d[:n].copy_(h[a:b], non_blocking=True)
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
                for h, d in zip(self.outputs, self.results[buf]):
                    h[a:b].copy_(d[:n], non_blocking=True)
                copied[buf] = torch.cuda.Event()
                copied[buf].record(self.d2h)
        for s in (self.h2d, self.compute, self.d2h):
            cur.wait_stream(s)
        return tuple(self.outputs)


def attention_fwd_bwd_host(q, k, v, dout, *, causal=False, block_causal=0, scale=None, device="cuda", slices=None,
                           pipeline=None):
    """out, dq, dk, dv (pinned host tensors) of ``attention(q, k, v, ...)`` and its backward for ``dout``.
    All four inputs: pinned host ``[B, H, S, D]`` views with a contiguous last dim (e.g. ``[B, S, H, D]``
    storage), fp16 or bf16, head dim 64 or 128. ``pipeline``: a ``HostPipeline`` to reuse buffers and
    streams across calls. The returned host tensors are valid once the current stream has caught up
    (``torch.cuda.current_stream().synchronize()``)."""
    if causal and block_causal not in (0, 1):
        raise ValueError("causal is block_causal=1: give one of them")
    block = 1 if causal else int(block_causal)
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    pipe = pipeline or HostPipeline(q, k, v, device, slices)
    return pipe.run(q, k, v, dout, scale, block)
