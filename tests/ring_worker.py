"""Multi-process check of kohakufa_b200.ring on real GPUs (one process per GPU, NCCL):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29544 tests/ring_worker.py [--seq 8192] [--dim 128]

Every rank builds the same seeded full-length inputs on the CPU, keeps its zig-zag shard, runs
ring_attention forward + backward, and rank 0 gathers the pieces and compares them with the single-GPU
kernels on the whole sequence and with the fp64 oracle. NVLS is not needed: plain send / recv."""
import argparse
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from kohakufa_b200 import _lib, attention, ring  # noqa: E402
from oracle import reference as oracle  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--heads", type=int, default=4)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, pg_options=ring.nccl_options())
    rank, world = dist.get_rank(), dist.get_world_size()
    dtype = torch.bfloat16
    gen = torch.Generator().manual_seed(7)
    full = [(torch.randn(1, args.seq, args.heads, args.dim, generator=gen) * 0.5).to(dtype).transpose(1, 2) for _ in range(4)]
    q, k, v, dout = (ring.zigzag_shard(x, rank, world).to(dev) for x in full)
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    for _ in range(2):  # twice: buffers and communicators warm, results must repeat
        for t in (q, k, v):
            t.grad = None
        out = ring.ring_attention(q, k, v)
        out.backward(dout)
    torch.cuda.synchronize()
    assert _lib.device_status(dev) == 0
    pieces = []
    for t in (out.detach(), q.grad, k.grad, v.grad):
        t = t.contiguous()
        bucket = [torch.empty_like(t) for _ in range(world)] if rank == 0 else None
        dist.gather(t, bucket, dst=0)
        pieces.append(bucket)
    if rank == 0:
        got = [ring.zigzag_unshard(p) for p in pieces]
        fq, fk, fv, fdo = (x.to(dev) for x in full)
        fq, fk, fv = (t.requires_grad_() for t in (fq, fk, fv))
        single = attention(fq, fk, fv, causal=True)
        single.backward(fdo)
        want = oracle.attention_fp64(fq, fk, fv, fdo, args.dim**-0.5, block=1)
        for name, g, s1, w in zip(("out", "dq", "dk", "dv"), got, (single, fq.grad, fk.grad, fv.grad), want):
            err, err1 = oracle.metrics(g, w)["rel_err"], oracle.metrics(s1, w)["rel_err"]
            print(f"ring N={world} S={args.seq} {name}: rel_err {err:.3e} (single call {err1:.3e})")
            assert err < 2e-2 and err <= 1.25 * err1 + 1e-5, name
        print("ring worker ok")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
