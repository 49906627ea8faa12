"""Worker of tests/test_ring.py::test_ring_shift_over_gloo_world_2 (run under torchrun, gloo, CPU)."""
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from kohakufa_b200 import ring  # noqa: E402

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
cur = torch.full((4,), float(rank))
nxt = torch.empty_like(cur)
acc = torch.zeros(3)
acc_in = torch.empty_like(acc)
acc_reqs = []
for t in range(world):
    reqs = ring._shift(cur, nxt, None) if t + 1 < world else []
    assert float(cur[0]) == (rank - t) % world
    if acc_reqs:
        ring._wait(acc_reqs)
        acc, acc_in = acc_in, acc
    acc += 10.0**rank
    acc_reqs = ring._shift(acc, acc_in, None)
    if reqs:
        ring._wait(reqs)
        cur, nxt = nxt, cur
ring._wait(acc_reqs)
acc = acc_in
assert float(acc[0]) == sum(10.0**r for r in range(world)), acc
print("ring ok", rank)
dist.destroy_process_group()
