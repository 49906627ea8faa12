"""Benchmark of the attention forward + backward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C3] [--impl ours|reference]

One step = one forward + backward of the named configuration (default C3: token-causal, bf16,
B=4, H=32, S=8192, D=128) through the torch custom ops, inputs resident in HBM. With N > 1 GPUs
(launched by ``python -m torch.distributed.run``) every rank runs the same configuration on its own
batch shard (batch x heads sharding, no communication; global batch = N x B), the timed region is
bracketed by barriers, and the step time is the maximum over ranks.

Rank 0 prints ONE JSON line: the metric (fwd+bwd TFLOP/s, algorithmic FLOPs in the reference's
convention), the end-to-end number through ``kohakufa_b200.attention`` with host buffers, the
tensor-core roofline of the dominant kernel from CUDA-event timings of each kernel inside the timed
steps, the CPU baseline (the fp64 oracle on the host cores, on a bounded sample), and the clocks
sampled during the timed region.

``--impl reference`` times the reference's CPU path (its fp64 oracle, restated in oracle/) on the
host cores instead, on a bounded sample of the same configuration.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "fwd+bwd TFLOP/s"
UNIT = "TFLOP/s"


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.first = 0  # rows before this index were sampled before the timed region began

    def wait_running(self, timeout=5.0):
        """Blocks until nvidia-smi has delivered its first row (it can take longer to start than a short
        timed region lasts), then marks where the region's own samples begin."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.rows and time.perf_counter() - t0 < timeout:
            time.sleep(0.02)
        self.first = len(self.rows)

    def samples_under_load(self):
        return len(self.rows) - self.first

    def __enter__(self):
        if self.index < 0:  # only rank 0 samples (its own GPU)
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL,
                text=True,
            )
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        clocks, reasons, max_mhz = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows[self.first :]:
            if len(row) < 7:
                continue
            try:
                clocks.append(float(row[0]))
                max_mhz = float(row[1])
            except ValueError:
                continue
            for name, val in zip(names, row[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {
            "sm_mhz": statistics.median(clocks),
            "sm_max_mhz": max_mhz,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def cpu_baseline(cfg, threads=None, target_seconds=12.0):
    """The fp64 oracle (forward + backward) on the host cores on a bounded sample of ``cfg``: one
    (batch, head) slice at the configuration's length capped so that the fp64 score matrices fit
    comfortably; repeated until about ``target_seconds`` have passed."""
    from kohakufa_b200 import workloads
    from oracle import reference as oracle

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    seq = min(cfg.seq, 4096)
    q, k, v, dout = workloads.make_inputs(cfg, batch=1, heads=1, seq=seq)
    flops = workloads.attention_flops(1, 1, seq, seq, cfg.dim, cfg.block)
    oracle.attention_fp64(q, k, v, dout, cfg.scale, cfg.block)  # warm-up
    reps, t0 = 0, time.perf_counter()
    while True:
        oracle.attention_fp64(q, k, v, dout, cfg.scale, cfg.block)
        reps += 1
        elapsed = time.perf_counter() - t0
        if elapsed > target_seconds or reps >= 50:
            break
    return {
        "value": flops * reps / elapsed / 1e12,
        "unit": UNIT,
        "cores": threads,
        "kind": "port",
        "sample": f"fp64 oracle, fwd+bwd, 1 batch x 1 head of {cfg.name} at S={seq}, {reps} repetitions in {elapsed:.1f} s",
    }


def run_reference(args, cfg):
    """The reference arm: its CPU path (fp64 attention of its tests/reference.py, restated in
    oracle/reference.py) on all host cores; each step is one bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from kohakufa_b200 import workloads
    from oracle import reference as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    seq = min(cfg.seq, 2048)
    q, k, v, dout = workloads.make_inputs(cfg, batch=1, heads=2, seq=seq)
    flops = workloads.attention_flops(1, 2, seq, seq, cfg.dim, cfg.block)
    for _ in range(args.warmup):
        oracle.attention_fp64(q, k, v, dout, cfg.scale, cfg.block)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.attention_fp64(q, k, v, dout, cfg.scale, cfg.block)
    elapsed = time.perf_counter() - t0
    value = flops * args.steps / elapsed / 1e12
    sample = f"fp64 oracle, fwd+bwd, 1 batch x 2 heads of {cfg.name} at S={seq} per step"
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f64",
        "data": "synthetic",
        "config": config_dict(cfg, 1) | {"sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def config_dict(cfg, n_gpus):
    mode = "dense" if cfg.block == 0 else ("token-causal" if cfg.block == 1 else f"block-causal P={cfg.block}")
    return {
        "workload": f"{cfg.name}: {mode} attention fwd+bwd, B={cfg.batch} H={cfg.heads} S={cfg.seq} D={cfg.dim} per GPU",
        "global_batch": cfg.batch if cfg.name.startswith("C5") else cfg.batch * n_gpus,
        "seq_len": cfg.seq,
        "parallelism": (
            f"context-parallel K/V ring over {n_gpus} GPUs (zig-zag sequence shards, NCCL send/recv)"
            if cfg.name.startswith("C5") and n_gpus > 1
            else f"batch x heads sharding over {n_gpus} GPU(s), no communication"
        ),
        "l2": l2_note(cfg),
    }


def l2_note(cfg):
    """How the timed steps relate to the 126 MB L2 (inputs of one step: q, k, v, dout)."""
    mb = 4 * cfg.batch * cfg.heads * cfg.seq * cfg.dim * 2 / 1e6
    if mb > 126:
        return f"inputs larger than L2 (4 tensors, {mb:.0f} MB per step); no flush needed"
    return f"inputs {mb:.1f} MB per step fit in L2 and are not flushed: a launch-bound parity configuration, not a roofline one"


# The reference's own published fwd+bwd TFLOP/s for a configuration's exact shape, where there is one
# (on B300, its only published hardware: benchmarks/results/speed.csv:202-203).
PUBLISHED = {"C4": 763.0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="C3")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="override the configuration's batch (profiling a small case)")
    ap.add_argument("--heads", type=int, default=None, help="override the configuration's head count")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from kohakufa_b200 import workloads

    cfg = workloads.CONFIGS[args.config]
    if args.batch or args.heads:
        import dataclasses

        cfg = dataclasses.replace(cfg, batch=args.batch or cfg.batch, heads=args.heads or cfg.heads)
    if args.impl == "reference":
        run_reference(args, cfg)
        return

    import torch.distributed as dist

    from kohakufa_b200 import _lib, attention
    from kohakufa_b200.op import attention_bwd_op, attention_fwd_op

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- inputs: this rank's batch shard, generated on the CPU, resident in HBM ----
    # C5 (one 131072-token sequence): context-parallel ring over the N GPUs, strong scaling.
    ring_mode = cfg.name.startswith("C5") and world > 1
    if cfg.name.startswith("C5"):
        chunk = cfg.seq // (2 * world)
        mine = sorted({rank, 2 * world - 1 - rank}) if ring_mode else [0, 1]
        host = workloads.make_piecewise_inputs(cfg, [(c * chunk, (c + 1) * chunk) for c in mine])
    else:
        host = workloads.make_inputs(cfg, seed_offset=rank)
    host = [t.transpose(1, 2).contiguous().pin_memory() for t in host]  # [B, S, H, D] storage
    q, k, v, dout = (t.to(dev, non_blocking=True).transpose(1, 2) for t in host)
    torch.cuda.synchronize()
    flops = workloads.attention_flops(cfg.batch, cfg.heads, cfg.seq, cfg.seq, cfg.dim, cfg.block)
    fwd_flops = flops / 3.5
    scale, block = cfg.scale, cfg.block

    if ring_mode:
        from kohakufa_b200 import ring

        def step():
            out, lse = ring.ring_forward(q, k, v, scale)
            return ring.ring_backward(q, k, v, out, dout, lse, scale)

    else:

        def step():
            out, lse = attention_fwd_op(q, k, v, scale, block)
            return attention_bwd_op(q, k, v, out, dout, lse, scale, block)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    assert _lib.device_status(dev) == 0, "a kernel wait timed out during warm-up"

    # ---- timed region: exactly K steps, device time, max over ranks ----
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local if rank == 0 else -1) as sampler:
        sampler.wait_running()
        barrier()
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        barrier()
        # per-kernel device times, same workload, still inside the sampled region
        kernel_ms = time_kernels(cfg, q, k, v, dout, args.steps)
        # a short timed region can end before nvidia-smi's next sample: keep the same load running
        # (untimed) until three samples under load exist, for at most 1.5 s
        t_extra = time.perf_counter()
        while rank == 0 and not ring_mode and sampler.samples_under_load() < 3 and time.perf_counter() - t_extra < 1.5:
            step()
            torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    # ring: all ranks work on ONE problem (strong scaling); otherwise every rank has its own copy
    value = (1 if ring_mode else world) * flops / (ms_per_step * 1e-3) / 1e12
    assert _lib.device_status(dev) == 0, "a kernel wait timed out during the timed region"

    # ---- end to end: host buffers in, host buffers out, through the public API ----
    e2e = None
    if not args.no_e2e:
        if ring_mode:
            attn = lambda a, b, c, **kw: ring.ring_attention(a, b, c, scale=scale)  # noqa: E731
            e2e = end_to_end(cfg, host, dev, attn, 1, flops, max(2, args.steps // 4), barrier, reduce_max=True)
        else:
            e2e = end_to_end(cfg, host, dev, attention, world, flops, max(3, args.steps // 4), barrier)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    units = {"fwd": 2, "dkdv": 4, "dq": 1}  # matmuls of the algorithmic count each kernel delivers
    dominant = max(("fwd", "dkdv", "dq"), key=lambda n: kernel_ms[n])
    # the kernels were timed on this rank's local tensors (the whole problem unless ring mode)
    local_fwd_flops = workloads.attention_flops(q.shape[0], q.shape[1], q.shape[2], q.shape[2], cfg.dim, cfg.block, backward=False)
    achieved = units[dominant] * (local_fwd_flops / 2) / (kernel_ms[dominant] * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"]
    # DRAM traffic of the dK/dV kernel from the ncu capture of the same shape at 16 heads
    # (profiles/attention_kernels_c3_b1h16_ncu.md), scaled by the number of heads (it grows in proportion)
    traffic = None
    if dominant == "dkdv" and (cfg.seq, cfg.dim, cfg.block) == (8192, 128, 1) and not ring_mode:
        traffic = 176.8e6 / 16 * q.shape[0] * q.shape[1]
    line = {
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "strong" if ring_mode else "weak",
        "vs_baseline": (value / world / PUBLISHED[cfg.name]) if cfg.name in PUBLISHED else None,
        "dtype": "bf16" if cfg.dtype == torch.bfloat16 else "fp16",
        "data": "synthetic",
        "config": config_dict(cfg, world),
        "pct_of_peak": {
            "of_measured_sustained": value / world / peaks["bf16_tflops_sustained"],
            "of_measured_burst": value / world / peaks["bf16_tflops"],
            "of_nominal_2250": value / world / 2250.0,
            "peaks": peak_kind,
        },
        "kernel_ms": kernel_ms,
        "roofline": {
            "bound": "tensor",
            "kernel": {"fwd": "kfa_fwd_kernel", "dkdv": "kfa_bwd_dkdv_kernel", "dq": "kfa_bwd_dq_kernel"}[dominant],
            "achieved": achieved,
            "peak": peak,
            "unit": "TFLOP/s",
            "frac": achieved / peak,
            "traffic": traffic,
            "note": f"algorithmic matmuls counted for this kernel: {units[dominant]} of 7; peak = {peak_kind} sustained cuBLAS bf16",
        },
        "gpu_launches": (3 * world + 5 if ring_mode else 4) * args.steps,
        "clocks": sampler.summary(),
        "e2e": e2e,
    }
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(cfg)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def time_kernels(cfg, q, k, v, dout, reps):
    """Average device time of each kernel of one step, CUDA events on the launching stream."""
    import ctypes

    from kohakufa_b200 import _lib
    from kohakufa_b200.op import attention_fwd_op

    lib = _lib.load()
    dev = q.device
    scale, block = cfg.scale, cfg.block
    out, lse = attention_fwd_op(q, k, v, scale, block)
    like = lambda t: t.new_empty(t.shape[0], t.shape[2], t.shape[1], t.shape[3]).transpose(1, 2)  # noqa: E731
    dq, dk, dv = like(q), like(k), like(v)
    stats = q.new_empty(lib.kfa_bwd_stats_bytes(q.shape[0], q.shape[1], q.shape[2]) // 4, dtype=torch.float32)
    T = {n: ctypes.byref(_lib.tensor4(t)) for n, t in dict(q=q, k=k, v=v, out=out, dout=dout, dq=dq, dk=dk, dv=dv).items()}
    code = _lib.dtype_code(q.dtype)
    word = _lib.status_word(dev).data_ptr()
    stream = _lib.stream_ptr(dev)
    calls = {
        "fwd": lambda: lib.kfa_fwd(T["q"], T["k"], T["v"], T["out"], lse.data_ptr(), scale, block, code, word, stream),
        "prepare": lambda: lib.kfa_bwd_prepare(T["out"], T["dout"], lse.data_ptr(), stats.data_ptr(), code, stream),
        "dkdv": lambda: lib.kfa_bwd_dkdv(T["q"], T["k"], T["v"], T["dout"], stats.data_ptr(), T["dk"], T["dv"], scale, block, code, word, stream),
        "dq": lambda: lib.kfa_bwd_dq(T["q"], T["k"], T["v"], T["dout"], stats.data_ptr(), T["dq"], scale, block, code, word, stream),
    }
    reps = max(3, min(reps, 10))
    events = {n: [] for n in calls}
    for _ in range(reps):
        for name, call in calls.items():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            _lib.check(call())
            b.record()
            events[name].append((a, b))
    torch.cuda.synchronize()
    return {n: sum(a.elapsed_time(b) for a, b in ev) / len(ev) for n, ev in events.items()}


def end_to_end(cfg, host, dev, attention, world, flops, steps, barrier, reduce_max=False):
    """The same metric through ``kohakufa_b200.attention`` with HOST buffers: every step copies q, k,
    v, dout from pinned host memory, runs forward + backward, and copies out, dq, dk, dv back."""
    hq, hk, hv, hdo = host
    if reduce_max:  # ring mode: one sequence over all ranks, no batch to pipeline over
        outs = [torch.empty_like(hq).pin_memory() for _ in range(4)]

        def step():
            q, k, v, dout = (t.to(dev, non_blocking=True).transpose(1, 2) for t in (hq, hk, hv, hdo))
            q, k, v = (t.requires_grad_() for t in (q, k, v))
            out = attention(q, k, v, causal=(cfg.block == 1), block_causal=0 if cfg.block == 1 else cfg.block)
            dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
            for dst, src in zip(outs, (out, dq, dk, dv)):
                dst.copy_(src.transpose(1, 2), non_blocking=True)

    else:  # the host-buffer entry point: batch slices pipelined over copy-in / compute / copy-out streams
        from kohakufa_b200 import hostio

        views = [t.transpose(1, 2) for t in (hq, hk, hv, hdo)]
        pipe = hostio.HostPipeline(*views[:3], dev)

        def step():
            hostio.attention_fwd_bwd_host(*views, causal=(cfg.block == 1), block_causal=0 if cfg.block == 1 else cfg.block,
                                          scale=cfg.scale, pipeline=pipe)

    for _ in range(3):
        step()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    barrier()
    ms = start.elapsed_time(stop)
    if world > 1 or reduce_max:
        import torch.distributed as dist

        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    nbytes = sum(t.numel() * t.element_size() for t in host)
    return {
        "value": world * flops / (ms / steps * 1e-3) / 1e12,
        "unit": UNIT,
        "ms_per_step": ms / steps,
        "steps": steps,
        "h2d_bytes_per_step": nbytes,
        "d2h_bytes_per_step": nbytes,
    }


if __name__ == "__main__":
    main()
