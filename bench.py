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
sampled during the timed region. Configurations whose step lasts microseconds (C1, C2) are timed as
one CUDA graph of the K steps, as the reference's benchmark does (benchmarks/speed.py:29-61): eager
launches would measure the host's launch rate instead of the kernels.

With N > 1 GPUs the line also carries a ``ring`` record: the context-parallel C5 problem (one causal
sequence of 131072 tokens spread over the N GPUs, strong scaling) timed the same way, with the share of
the step the compute stream spent waiting for NCCL, the ring's results against the single-GPU kernels
at S = 16384, and fp64 spot checks of rows of the full-length result.

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


def reference_sample(cfg):
    """The bounded sample of ``cfg`` both CPU measurements run: 1 batch x 2 heads at the configuration's
    length capped at 2048 (fp64 score matrices of a longer slice would not be a few seconds of work)."""
    from kohakufa_b200 import workloads

    seq = min(cfg.seq, 2048)
    inputs = workloads.make_inputs(cfg, batch=1, heads=2, seq=seq)
    flops = workloads.attention_flops(1, 2, seq, seq, cfg.dim, cfg.block)
    return inputs, flops, f"fp64 oracle, fwd+bwd, 1 batch x 2 heads of {cfg.name} at S={seq}"


def cpu_baseline(cfg, threads=None, target_seconds=12.0):
    """The fp64 oracle (forward + backward) on the host cores on the bounded sample of ``cfg``, repeated
    until about ``target_seconds`` have passed."""
    from oracle import reference as oracle

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    (q, k, v, dout), flops, sample = reference_sample(cfg)
    oracle.attention_fp64(q, k, v, dout, cfg.scale, cfg.block)  # warm-up
    reps, t0 = 0, time.perf_counter()
    while True:
        oracle.attention_fp64(q, k, v, dout, cfg.scale, cfg.block)
        reps += 1
        elapsed = time.perf_counter() - t0
        if elapsed > target_seconds or reps >= 200:
            break
    return {
        "value": flops * reps / elapsed / 1e12,
        "unit": UNIT,
        "cores": threads,
        "kind": "port",
        "sample": f"{sample}, {reps} repetitions in {elapsed:.1f} s",
    }


def run_reference(args, cfg):
    """The reference arm: its CPU path (fp64 attention of its tests/reference.py, restated in
    oracle/reference.py) on all host cores; each step is one bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import reference as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    (q, k, v, dout), flops, sample = reference_sample(cfg)
    sample += " per step"
    for _ in range(args.warmup):
        oracle.attention_fp64(q, k, v, dout, cfg.scale, cfg.block)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.attention_fp64(q, k, v, dout, cfg.scale, cfg.block)
    elapsed = time.perf_counter() - t0
    value = flops * args.steps / elapsed / 1e12
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
        "config": config_dict(cfg, args.gpus),
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
    ap.add_argument("--head-dim", type=int, default=None, help="override the configuration's head dim (a multiple of 16 up to 128)")
    ap.add_argument("--backward", default=None, choices=["auto", "fused", "split"],
                    help="backward implementation (default: the package's, 'auto' unless KFA_BACKWARD says otherwise)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-ring", action="store_true", help="N > 1: skip the context-parallel C5 record")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from kohakufa_b200 import workloads

    cfg = workloads.CONFIGS[args.config]
    if args.batch or args.heads or args.head_dim:
        import dataclasses

        cfg = dataclasses.replace(cfg, batch=args.batch or cfg.batch, heads=args.heads or cfg.heads,
                                  dim=args.head_dim or cfg.dim)
    if args.impl == "reference":
        run_reference(args, cfg)
        return

    import torch.distributed as dist

    from kohakufa_b200 import _lib, attention, get_backward, set_backward
    from kohakufa_b200.op import attention_bwd_op, attention_fwd_op, use_fused_backward

    if args.backward:
        set_backward(args.backward)
    fused = use_fused_backward(cfg.dim, cfg.batch * cfg.heads)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    affinity = bind_to_gpu_cpus(local)  # before any pinned allocation: first touch places the pages
    if world > 1:
        from kohakufa_b200.ring import nccl_options

        dist.init_process_group("nccl", device_id=dev, pg_options=nccl_options())  # (the C5 ring record uses it)

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

    # A step of a few hundred microseconds is launch-bound when issued eagerly: such configurations are
    # timed as ONE CUDA graph holding the K steps (the reference's method, benchmarks/speed.py:29-61).
    use_graph = (not ring_mode) and flops < 1e11
    graph = None
    if use_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(args.steps):
                    step()
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()  # one untimed replay
        barrier()

    # ---- timed region: exactly K steps, device time, max over ranks ----
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local if rank == 0 else -1) as sampler:
        sampler.wait_running()
        barrier()
        start.record()
        if graph is not None:
            graph.replay()
        else:
            for _ in range(args.steps):
                step()
        stop.record()
        barrier()
        # per-kernel device times, same workload, still inside the sampled region
        kernel_ms = time_kernels(cfg, q, k, v, dout, args.steps, not fused)
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
        e2e["cpu_affinity"] = affinity

    # ---- N > 1: the context-parallel ring on C5, under the same launch ----
    ring_rec = None
    if world > 1 and not ring_mode and not args.no_ring:
        del q, k, v, dout, host
        torch.cuda.empty_cache()
        ring_rec = ring_record(rank, world, dev, barrier)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    # matmuls of the algorithmic count (2 forward + 5 backward) each kernel delivers; the split dQ kernel's
    # S and dP are recomputation and count for nothing
    units = {"fwd": 2, "fused": 5, "dkdv": 4, "dq": 1}
    names = {"fwd": "kfa_fwd_kernel", "fused": "kfa_bwd_fused_kernel", "dkdv": "kfa_bwd_dkdv_kernel", "dq": "kfa_bwd_dq_kernel"}
    dominant = max((n for n in units if n in kernel_ms), key=lambda n: kernel_ms[n])
    # the kernels were timed on this rank's local tensors (the whole problem unless ring mode)
    local_rows = cfg.seq // world if ring_mode else cfg.seq
    local_fwd_flops = workloads.attention_flops(cfg.batch, cfg.heads, local_rows, local_rows, cfg.dim, cfg.block, backward=False)
    achieved = units[dominant] * (local_fwd_flops / 2) / (kernel_ms[dominant] * 1e-3) / 1e12
    clocks = sampler.summary()
    # 4096 multiply-adds per clock and SM at the clock the GPU actually ran the timed region at
    clock_peak = 4096 * 2 * 148 * clocks["sm_mhz"] * 1e6 / 1e12 if clocks.get("sm_mhz") else None
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
        "config": config_dict(cfg, world)
        | {"timing": f"one CUDA graph of {args.steps} steps" if use_graph else "eager launches, CUDA events"}
        | {"backward": f"{'fused kernel' if fused else 'split kernels'} (mode {get_backward()})"},
        "pct_of_peak": {
            "of_measured_burst": value / world / peaks["bf16_tflops"],
            "of_measured_sustained": value / world / peaks["bf16_tflops_sustained"],
            "of_nominal_2250": value / world / 2250.0,
            "peaks": peak_kind,
        },
        "kernel_ms": kernel_ms,
        "roofline": {
            "bound": "tensor",
            "kernel": names[dominant],
            "achieved": achieved,
            "peak": peaks["bf16_tflops"],
            "unit": "TFLOP/s",
            "frac": achieved / peaks["bf16_tflops"],
            "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"],
            "frac_of_clock_normalised_peak": achieved / clock_peak if clock_peak else None,
            "traffic": ncu_traffic(dominant, cfg, q_heads=cfg.batch * cfg.heads) if not ring_mode else None,
            "note": f"algorithmic matmuls counted for this kernel: {units[dominant]} of 7; peak = {peak_kind} burst cuBLAS bf16 "
            "(the timed region lasts a fraction of a second); sustained = the same GEMM in a seconds-long loop; "
            "clock-normalised = 4096 MAC x 2 x 148 SMs x the median SM clock sampled during the timed region; "
            "traffic = DRAM bytes of one launch from an ncu capture of a small case of the same shape, scaled by the (batch, head) pairs",
        },
        "gpu_launches": (3 * world + 5 if ring_mode else 4) * args.steps,  # fwd + 3 backward launches either way
        "clocks": clocks,
        "e2e": e2e,
    }
    if ring_rec is not None:
        line["ring"] = ring_rec
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(cfg)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of a kernel, from ncu captures of a
# small case of the configuration's shape: (kernel, S, D, block) -> (bytes, (batch, head) pairs of the
# captured launch). A launch's traffic grows in proportion to the pairs, so a full launch is scaled by them.
NCU_DRAM_BYTES = {
    ("dkdv", 8192, 128, 1): (173.8e6, 16),
    ("dq", 8192, 128, 1): (157.1e6, 16),
    ("fwd", 8192, 128, 1): (114.8e6, 16),
    ("fused", 8192, 128, 1): (299.9e6, 16),
    ("fused", 4096, 64, 256): (294.7e6, 64),
    ("fwd", 4096, 64, 256): (118.5e6, 64),
}


def ncu_traffic(kernel, cfg, q_heads):
    entry = NCU_DRAM_BYTES.get((kernel, cfg.seq, cfg.dim, cfg.block))
    return None if entry is None else entry[0] / entry[1] * q_heads


def bind_to_gpu_cpus(index):
    """Pins this process to the CPU cores the driver reports as local to GPU ``index`` (NVML, read-only),
    so that the pinned host buffers allocated afterwards are placed on that NUMA node. Returns what was
    done, for the record."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        allowed = os.sched_getaffinity(0)
        use = sorted(cpus & allowed)
        if use and len(use) < len(allowed):
            os.sched_setaffinity(0, use)
            return {"bound_to": f"{use[0]}-{use[-1]} ({len(use)} of {len(allowed)} allowed cores)", "source": "NVML"}
        return {"bound_to": None, "note": f"GPU-local cores ({len(cpus)}) cover all {len(allowed)} allowed cores: one NUMA domain visible"}
    except Exception as exc:  # no NVML, or a cpuset that forbids it: run unbound
        return {"bound_to": None, "note": f"affinity not set: {type(exc).__name__}"}


def time_kernels(cfg, q, k, v, dout, reps, deterministic=False):
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
    calls = {"fwd": lambda: lib.kfa_fwd(T["q"], T["k"], T["v"], T["out"], lse.data_ptr(), scale, block, code, word, stream)}
    if deterministic:
        calls |= {
            "prepare": lambda: lib.kfa_bwd_prepare(T["out"], T["dout"], lse.data_ptr(), stats.data_ptr(), code, stream),
            "dkdv": lambda: lib.kfa_bwd_dkdv(T["q"], T["k"], T["v"], T["dout"], stats.data_ptr(), T["dk"], T["dv"], scale, block, code, word, stream),
            "dq": lambda: lib.kfa_bwd_dq(T["q"], T["k"], T["v"], T["dout"], stats.data_ptr(), T["dq"], scale, block, code, word, stream),
        }
    else:
        acc = q.new_empty(lib.kfa_bwd_dq_acc_bytes(*q.shape) // 4, dtype=torch.float32)
        calls |= {
            "prepare": lambda: lib.kfa_bwd_prepare_fused(T["out"], T["dout"], lse.data_ptr(), stats.data_ptr(), acc.data_ptr(), code, stream),
            "fused": lambda: lib.kfa_bwd_fused_main(T["q"], T["k"], T["v"], T["dout"], stats.data_ptr(), acc.data_ptr(), T["dk"], T["dv"], scale, block, code, word, stream),
            "convert": lambda: lib.kfa_bwd_dq_convert(acc.data_ptr(), T["dq"], scale, code, word, stream),
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


def ring_record(rank, world, dev, barrier, steps=2):
    """The context-parallel ring on C5 (causal bf16, B=1, H=32, S=131072, D=128 spread zig-zag over the
    ``world`` GPUs), measured and checked under the same launch as the main line:

    * ``value`` / ``ms_per_step``: forward + backward of the WHOLE problem (strong scaling), device time, max
      over ranks; ``stream_ms``: where the compute stream's time went on the slowest rank (kernels against
      stalls waiting for NCCL transfers), from events around every wait;
    * ``parity_s16384``: the ring's out / dQ / dK / dV at S = 16384 against the single-GPU kernels on the same
      tensors (relative L2 distance, max over ranks; both are bf16 roundings of fp32 sums taken in a
      different order, so they differ by single bf16 roundings: the bound is 2^-8);
    * ``fp64_spot_checks``: at the full length, 4 heads x (first, middle, last) 512 query rows of out and dQ,
      and dK / dV of the last 512 keys, against a chunk-free fp64 evaluation of those rows (relative L2
      error; the tolerance is the bf16 one of the tests, 2e-2).
    The inputs are drawn on the device (seeded per 8192-row piece): the checks are computed from the very
    tensors the kernels read."""
    import torch.distributed as dist

    from kohakufa_b200 import ring, workloads
    from kohakufa_b200.op import attention_bwd_op, attention_fwd_op

    cfg = workloads.CONFIGS["C5"]
    scale = cfg.scale

    def my_ranges(seq):
        chunk = seq // (2 * world)
        return [(c * chunk, (c + 1) * chunk) for c in sorted({rank, 2 * world - 1 - rank})]

    def shard_only(seq):  # this rank's rows, generated piece by piece (chunks are whole pieces)
        return workloads.make_piecewise_inputs(cfg, my_ranges(seq), device=dev, device_rng=True)

    def shard_and_full(seq):  # a short sequence: every rank builds all of it and cuts its rows out
        full = workloads.make_piecewise_inputs(cfg, [(0, seq)], device=dev, device_rng=True)
        return tuple(ring.zigzag_shard(t, rank, world) for t in full), full

    def rel(got, want):
        return float((got.double() - want.double()).norm() / want.double().norm().clamp_min(1e-300))

    def reduce_max(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rec = {"workload": f"C5: token-causal bf16 B=1 H={cfg.heads} S={cfg.seq} D={cfg.dim}, zig-zag shards over {world} GPUs"}

    # ---- (1) parity with the single-GPU kernels at S = 16384 ----
    small = 16384
    (q, k, v, dout), full = shard_and_full(small)
    out, lse = ring.ring_forward(q, k, v, scale)
    dq, dk, dv = ring.ring_backward(q, k, v, out, dout, lse, scale)
    fq, fk, fv, fdo = full
    fout, flse = attention_fwd_op(fq, fk, fv, scale, 1)
    fgrads = attention_bwd_op(fq, fk, fv, fout, fdo, flse, scale, 1)
    rec["parity_s16384"] = {
        name: reduce_max(rel(got, ring.zigzag_shard(want, rank, world)))
        for name, got, want in zip(("out", "dq", "dk", "dv"), (out, dq, dk, dv), (fout, *fgrads))
    }
    del q, k, v, dout, full, out, lse, dq, dk, dv, fq, fk, fv, fdo, fout, flse, fgrads
    torch.cuda.empty_cache()

    # ---- (2) the full length: timing with a per-wait breakdown ----
    q, k, v, dout = shard_only(cfg.seq)

    def step(trace=None):
        out, lse = ring.ring_forward(q, k, v, scale, trace=trace)
        return out, lse, ring.ring_backward(q, k, v, out, dout, lse, scale, trace=trace)

    for _ in range(2):  # warm-up: communicators, allocator
        step()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    barrier()
    ms = reduce_max(start.elapsed_time(stop)) / steps
    flops = workloads.attention_flops(cfg.batch, cfg.heads, cfg.seq, cfg.seq, cfg.dim, cfg.block)
    rec |= {"value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "steps": steps, "scaling": "strong"}
    trace = []
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    out, lse, (dq, dk, dv) = step(trace)
    b.record()
    barrier()
    parts = ring.trace_summary(trace)
    parts["whole step"] = a.elapsed_time(b)
    parts["other (packing, finalize, prepare)"] = parts["whole step"] - sum(v_ for k_, v_ in parts.items() if k_ != "whole step")
    # report the slowest rank's breakdown
    mine = torch.tensor([parts["whole step"], float(rank)], device=dev, dtype=torch.float64)
    every = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    slowest = int(max(every, key=lambda t: float(t[0]))[1].item())
    keys = sorted(parts)
    vals = torch.tensor([parts[k_] for k_ in keys], device=dev, dtype=torch.float64)
    dist.broadcast(vals, src=slowest)
    rec["stream_ms"] = {"rank": slowest} | {k_: float(x) for k_, x in zip(keys, vals)}

    # ---- (3) fp64 spot checks of the full-length result ----
    heads = [0, cfg.heads // 3, 2 * cfg.heads // 3, cfg.heads - 1]
    c = cfg.seq // (2 * world)

    def gather_heads(t):  # this rank's rows of the chosen heads -> the whole sequence, [heads, S, D]
        mine = t[0, heads].contiguous()
        parts_ = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts_, mine)
        return ring.zigzag_unshard([p_.unsqueeze(0) for p_ in parts_])[0]

    K, V = gather_heads(k), gather_heads(v)
    # (global first row, local first row, owner) of the three 512-row blocks
    blocks = {"first": (0, 0, 0), "middle": (world * c - 256, c - 256, world - 1), "last": (cfg.seq - 512, 2 * c - 512, 0)}
    errs = {}
    for name, (g0, l0, owner) in blocks.items():
        worst = {"out": 0.0, "dq": 0.0}
        if name == "last":
            worst |= {"dk": 0.0, "dv": 0.0}
        if rank == owner:
            n_keys = g0 + 512
            for hi, h in enumerate(heads):
                qb, dob = q[0, h, l0 : l0 + 512].double(), dout[0, h, l0 : l0 + 512].double()
                kk, vv = K[hi, :n_keys].double(), V[hi, :n_keys].double()
                s_ = (qb @ kk.T) * scale
                cols = torch.arange(n_keys, device=dev)[None, :]
                s_.masked_fill_(cols > (g0 + torch.arange(512, device=dev))[:, None], float("-inf"))
                p_ = torch.softmax(s_, dim=-1)
                del s_
                o_ = p_ @ vv
                ds_ = p_ * (dob @ vv.T - (dob * o_).sum(-1, keepdim=True))
                worst["out"] = max(worst["out"], rel(out[0, h, l0 : l0 + 512], o_))
                worst["dq"] = max(worst["dq"], rel(dq[0, h, l0 : l0 + 512], ds_ @ kk * scale))
                if name == "last":  # only these 512 queries see the last 512 keys
                    worst["dk"] = max(worst["dk"], rel(dk[0, h, l0 : l0 + 512], ds_[:, g0:].T @ qb * scale))
                    worst["dv"] = max(worst["dv"], rel(dv[0, h, l0 : l0 + 512], p_[:, g0:].T @ dob))
                del p_, ds_, o_
        errs[name] = {k_: reduce_max(x) for k_, x in worst.items()}
    rec["fp64_spot_checks"] = {"heads": heads, "rows": 512, "rel_err": errs, "tolerance": 2e-2}
    rec["checks_pass"] = all(x < 2e-2 for blk in errs.values() for x in blk.values()) and all(
        x < 2.0**-8 for x in rec["parity_s16384"].values()
    )
    return rec


def copy_rates(host, dev, reps=3):
    """GB/s of the host-to-device and the device-to-host copy alone, with the bench's own pinned buffers."""
    dst = [torch.empty_like(t, device=dev) for t in host]
    nbytes = sum(t.numel() * t.element_size() for t in host)
    rates = {}
    for name, pairs in (("h2d_gbs", list(zip(dst, host))), ("d2h_gbs", list(zip(host, dst)))):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            for d, s_ in pairs:
                d.copy_(s_, non_blocking=True)
        b.record()
        torch.cuda.synchronize()
        rates[name] = nbytes * reps / (a.elapsed_time(b) * 1e-3) / 1e9
    return rates


def end_to_end(cfg, host, dev, attention, world, flops, steps, barrier, reduce_max=False):
    """The same metric through ``kohakufa_b200.attention`` with HOST buffers: every step copies q, k,
    v, dout from pinned host memory, runs forward + backward, and copies out, dq, dk, dv back. Also
    reports the two copy directions timed alone on every rank at once (the PCIe / host-memory bound)."""
    hq, hk, hv, hdo = host
    barrier()
    rates = copy_rates(host, dev)
    barrier()
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

        t = torch.tensor([ms, -rates["h2d_gbs"], -rates["d2h_gbs"]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0].item())
        rates = {"h2d_gbs": -float(t[1].item()), "d2h_gbs": -float(t[2].item())}
    nbytes = sum(t.numel() * t.element_size() for t in host)
    return {
        "value": world * flops / (ms / steps * 1e-3) / 1e12,
        "unit": UNIT,
        "ms_per_step": ms / steps,
        "steps": steps,
        "h2d_bytes_per_step": nbytes,
        "d2h_bytes_per_step": nbytes,
        "copy_only_per_rank": rates | {"note": "each direction alone, all ranks copying at once, slowest rank"},
    }


if __name__ == "__main__":
    main()
