"""Context-parallel ring attention: schedule logic on the CPU (incl. a world_size-2 gloo ring), and on a
GPU the full schedule with all ranks emulated in one process against the single-call kernels and the
fp64 oracle. The real multi-process run is tests/ring_worker.py under torchrun."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from kohakufa_b200 import ring

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_step_plan_covers_every_visible_chunk_pair_once(world):
    c = 256
    seen = {}
    for r in range(world):
        mine = (r, 2 * world - 1 - r)
        for t in range(world):
            src = (r - t) % world
            theirs = (src, 2 * world - 1 - src)
            block, (q0, q1), (k0, k1) = ring.step_plan(r, world, t, c)
            for qi in range(q0 // c, q1 // c):
                for ki in range(k0 // c, k1 // c):
                    pair = (mine[qi], theirs[ki])
                    kind = "causal" if block == 1 else "dense"
                    if block == 1 and qi > ki:
                        kind = "dense"  # below the diagonal of the local causal call
                    if block == 1 and qi < ki:
                        continue  # hidden inside the causal call
                    assert pair not in seen
                    seen[pair] = kind
    for a in range(2 * world):
        for b in range(2 * world):
            if b < a:
                assert seen.get((a, b)) == "dense", (a, b)
            elif b == a:
                assert seen.get((a, b)) == "causal", (a, b)
            else:
                assert (a, b) not in seen, (a, b)
    # balance: every rank does the same number of chunk pairs (diagonal ones count half)
    loads = []
    for r in range(world):
        load = 0.0
        for t in range(world):
            block, (q0, q1), (k0, k1) = ring.step_plan(r, world, t, c)
            area = (q1 - q0) * (k1 - k0) / c / c
            load += area * (0.5 if block else 1.0)  # the causal call covers 2 of its 4 chunk pairs
        loads.append(load)
    assert max(loads) == min(loads)


def test_zigzag_roundtrip():
    x = torch.arange(2 * 3 * 32 * 4, dtype=torch.float32).reshape(2, 3, 32, 4)
    for world in (1, 2, 4):
        parts = [ring.zigzag_shard(x, r, world) for r in range(world)]
        assert parts[0].transpose(1, 2).is_contiguous()
        assert torch.equal(ring.zigzag_unshard(parts), x)
    p0 = ring.zigzag_shard(x, 0, 4)
    assert torch.equal(p0[:, :, :4], x[:, :, :4]) and torch.equal(p0[:, :, 4:], x[:, :, 28:])


def test_local_shape_rules():
    q = torch.zeros(1, 2, 300, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="multiple of 256"):
        ring._check_local(q, q, q)
    q = torch.zeros(1, 2, 512, 64, dtype=torch.float32)
    with pytest.raises(TypeError):
        ring._check_local(q, q, q)


def test_ring_shift_over_gloo_world_2():
    """Two CPU processes (gloo): what each rank receives over N hops of `_shift` is what the schedule
    says it holds (the tensors of rank (r - t) mod N), and an accumulator that every rank adds to comes
    home complete after N hops (tests/gloo_ring_check.py)."""
    env = dict(os.environ, OMP_NUM_THREADS="1")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "gloo_ring_check.py")],
        capture_output=True, text=True, env=env, timeout=240,
    )
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert proc.stdout.count("ring ok") == 2


@pytest.mark.gpu
@pytest.mark.parametrize("world,dim,dtype", [(2, 128, torch.bfloat16), (4, 64, torch.float16), (4, 128, torch.bfloat16)])
def test_emulated_ring_matches_single_call_and_oracle(world, dim, dtype):
    from kohakufa_b200 import _lib, attention
    from oracle import reference as oracle

    seq = 2 * world * 256
    gen = torch.Generator().manual_seed(world)
    full = [(torch.randn(1, seq, 2, dim, generator=gen) * 0.7).to(dtype).cuda().transpose(1, 2) for _ in range(4)]
    q, k, v, dout = full
    shards = [[ring.zigzag_shard(x, r, world) for r in range(world)] for x in full]
    outs, lses, dqs, dks, dvs = ring.emulate_ring(*shards)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    got = [ring.zigzag_unshard(p) for p in (outs, dqs, dks, dvs)]
    # against the single-call kernels on the whole sequence
    ql, kl, vl = (x.clone().requires_grad_() for x in (q, k, v))
    ref_out = attention(ql, kl, vl, causal=True)
    ref_out.backward(dout)
    tol = 5e-3 if dtype == torch.float16 else 2e-2
    want = oracle.attention_fp64(q, k, v, dout, dim**-0.5, block=1)
    for name, g, single, w in zip(("out", "dq", "dk", "dv"), got, (ref_out, ql.grad, kl.grad, vl.grad), want):
        assert bool(torch.isfinite(g).all()), name
        err = oracle.metrics(g, w)["rel_err"]
        err_single = oracle.metrics(single, w)["rel_err"]
        assert err < tol, (name, err)
        assert err <= 1.25 * err_single + 1e-5, (name, err, err_single)  # no worse than one call


def test_nccl_options_ask_for_a_high_priority_stream():
    """The ring's transfers only overlap the attention grids when NCCL's kernels run at high priority."""
    if not hasattr(torch.distributed, "ProcessGroupNCCL"):
        pytest.skip("torch built without NCCL")
    assert ring.nccl_options().is_high_priority_stream

