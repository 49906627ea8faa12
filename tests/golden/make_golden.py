"""Generates the golden fixtures that pin ``oracle/reference.py`` to the reference's own code.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/KohakuFA

It imports the reference's ``tests/reference.py`` (fp64 attention + metrics) and
``benchmarks/dinov3_backward.py`` (``emulated_grads``, the correct-kernel rounding floor and its
bug variants), runs them on small seeded CPU inputs and stores inputs' recipe + outputs in
``tests/golden/*.npz``, plus ``floor_large_logit.json``: the error of the reference's emulated floor
against the reference's fp64 gradients on the large-logit workloads of ``kohakufa_b200.workloads`` (only
the error norms are stored, the tensors are regenerated from their seeds by the tests). The fixtures
travel with the repository; the reference does not.
"""

import json

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

# name -> (B, H, Sq, Skv, D, dtype, block, seed, input std)
ATTENTION_CASES = {
    "dense_f16": (2, 1, 40, 40, 64, "float16", 0, 11, 1.0),
    "causal_f16": (1, 2, 77, 77, 64, "float16", 1, 12, 1.0),
    "block7_f16": (1, 2, 50, 50, 32, "float16", 7, 13, 1.0),
    "causal_sq_lt_skv": (1, 2, 33, 70, 64, "float16", 1, 14, 1.0),
    "causal_sq_gt_skv": (1, 2, 70, 33, 64, "float16", 1, 15, 1.0),
    "block24_bf16": (1, 1, 61, 61, 128, "bfloat16", 24, 16, 0.5),
    "dense_cross_bf16": (1, 1, 19, 45, 128, "bfloat16", 0, 17, 1.0),
}
# Boolean masks and grouped-query attention: name -> (B, H, Hkv, Sq, Skv, D, dtype, seed, mask kind)
MASK_CASES = {
    "mask_random_f16": (2, 2, 2, 37, 45, 64, "float16", 31, "random"),
    "mask_broadcast_empty_rows_f16": (2, 3, 3, 40, 40, 32, "float16", 32, "empty_rows"),
    "mask_key_padding_bf16": (2, 2, 2, 30, 50, 64, "bfloat16", 33, "key_padding"),
    "gqa_causal_f16": (1, 4, 2, 33, 33, 64, "float16", 34, "causal_block"),
    "mask_gqa_bf16": (1, 4, 1, 29, 41, 64, "bfloat16", 35, "random"),
}


def make_mask_inputs(case):
    """q, k, v, dout, mask (None for the block-causal GQA case), block."""
    b, h, hkv, sq, skv, d, dtype, seed, kind = case
    gen = torch.Generator().manual_seed(seed)
    dt = getattr(torch, dtype)
    q = torch.randn(b, h, sq, d, generator=gen).to(dt)
    k = torch.randn(b, hkv, skv, d, generator=gen).to(dt)
    v = torch.randn(b, hkv, skv, d, generator=gen).to(dt)
    dout = torch.randn(b, h, sq, d, generator=gen).to(dt)
    if kind == "random":
        return q, k, v, dout, torch.rand(b, h, sq, skv, generator=gen) < 0.4, 0
    if kind == "empty_rows":  # one mask for every batch and head, rows 5..9 see nothing
        mask = torch.rand(1, 1, sq, skv, generator=gen) < 0.5
        mask[:, :, 5:10] = False
        return q, k, v, dout, mask, 0
    if kind == "key_padding":  # [B, 1, 1, Skv]: per-batch key lengths
        lengths = torch.tensor([skv, skv // 3])
        return q, k, v, dout, (torch.arange(skv)[None, :] < lengths[:, None])[:, None, None, :], 0
    return q, k, v, dout, None, 1


# name -> (B, H, S, D, dtype, seed, magnitude of q and k)
FLOOR_CASES = {
    "floor_f16": (1, 1, 40, 64, "float16", 21, 1.0),
    "floor_bf16": (1, 1, 40, 64, "bfloat16", 22, 1.0),
    "floor_large_f16": (1, 1, 40, 64, "float16", 23, 30.0),
    "floor_large_bf16": (1, 1, 40, 64, "bfloat16", 24, 30.0),
}
BUG_SETS = {"floor": (), "scale_ds": ("scale*dS",), "single_lse": ("single lse",), "scale_shift": ("scale-shift",)}
# The large-logit workloads the GPU floor tests run: name -> (generator, arguments)
LARGE_LOGIT_CASES = {
    "C2": ("config", "C2", 4),
    "C2-bf16": ("config", "C2-bf16", 4),
    "balanced-f16": ("balanced", "float16"),
    "balanced-bf16": ("balanced", "bfloat16"),
}


def make_large_logit_inputs(name):
    """q, k, v, dout ([B, H, S, D], CPU, already rounded) and the softmax scale of a LARGE_LOGIT_CASES entry."""
    sys.path.insert(0, str(HERE.parent.parent))
    from kohakufa_b200 import workloads

    case = LARGE_LOGIT_CASES[name]
    if case[0] == "config":
        cfg = workloads.CONFIGS[case[1]]
        return workloads.make_inputs(cfg, batch=case[2], heads=cfg.heads), cfg.scale
    return workloads.balanced_large_logit_inputs(1, 4, 512, 64, getattr(torch, case[1])), 64**-0.5


def make_attention_inputs(case):
    b, h, sq, skv, d, dtype, block, seed, std = case
    gen = torch.Generator().manual_seed(seed)
    dt = getattr(torch, dtype)
    q = (torch.randn(b, h, sq, d, generator=gen) * std).to(dt)
    k = (torch.randn(b, h, skv, d, generator=gen) * std).to(dt)
    v = (torch.randn(b, h, skv, d, generator=gen) * std).to(dt)
    dout = (torch.randn(b, h, sq, d, generator=gen) * std).to(dt)
    return q, k, v, dout


def make_floor_inputs(case):
    b, h, s, d, dtype, seed, mag = case
    gen = torch.Generator().manual_seed(seed)
    dt = getattr(torch, dtype)
    q = (torch.randn(b, h, s, d, generator=gen) * mag).to(dt)
    k = (torch.randn(b, h, s, d, generator=gen) * mag).to(dt)
    v = torch.randn(b, h, s, d, generator=gen).to(dt)
    dout = torch.randn(b, h, s, d, generator=gen).to(dt)
    return q, k, v, dout


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str) -> None:
    root = Path(ref_root)
    ref = _load(root / "tests" / "reference.py", "kfa_ref_oracle")
    out = {}
    for name, case in ATTENTION_CASES.items():
        q, k, v, dout = make_attention_inputs(case)
        scale = case[4] ** -0.5
        o, dq, dk, dv = ref.reference(q, k, v, dout, scale, block=case[6])
        for key, val in zip(("out", "dq", "dk", "dv"), (o, dq, dk, dv)):
            out[f"{name}/{key}"] = val.numpy()
        # the reference's metrics() on a perturbed copy, to pin metrics too
        noisy = o + 1e-3 * torch.randn(o.shape, generator=torch.Generator().manual_seed(5), dtype=torch.float64)
        m = ref.metrics(noisy, o)
        out[f"{name}/metrics"] = np.array([m["cos"], m["norm_ratio"], m["rel_err"], m["max_abs_err"], m["max_rel_err"]])
    for name, case in MASK_CASES.items():
        q, k, v, dout, mask, block = make_mask_inputs(case)
        o, dq, dk, dv = ref.reference(q, k, v, dout, case[5] ** -0.5, block=block, groups=case[1] // case[2], mask=mask)
        for key, val in zip(("out", "dq", "dk", "dv"), (o, dq, dk, dv)):
            out[f"{name}/{key}"] = val.numpy()
    np.savez_compressed(HERE / "attention_fp64.npz", **out)

    sys.path.insert(0, str(root / "benchmarks"))
    emu = _load(root / "benchmarks" / "dinov3_backward.py", "kfa_ref_emulation")
    out = {}
    for name, case in FLOOR_CASES.items():
        q, k, v, dout = make_floor_inputs(case)
        inputs = {"q": q, "k": k, "v": v, "dout": dout, "scale": case[3] ** -0.5}
        for tag, bugs in BUG_SETS.items():
            dq, dk, dv = emu.emulated_grads(inputs, set(bugs))
            for key, val in zip(("dq", "dk", "dv"), (dq, dk, dv)):
                out[f"{name}/{tag}/{key}"] = val.numpy()
    np.savez_compressed(HERE / "floor_emulation.npz", **out)

    def rel_l2(got, want):
        return float((got.double() - want.double()).norm() / want.double().norm())

    floors = {}
    for name in LARGE_LOGIT_CASES:
        (q, k, v, dout), scale = make_large_logit_inputs(name)
        want = ref.reference(q, k, v, dout, scale)[1:]
        inputs = {"q": q, "k": k, "v": v, "dout": dout, "scale": scale}
        entry = {}
        for tag, bugs in BUG_SETS.items():
            got = emu.emulated_grads(inputs, set(bugs))
            entry[tag] = {key: rel_l2(g, w) for key, g, w in zip(("dq", "dk", "dv"), got, want)}
            if tag == "floor":  # the same with the gradients themselves rounded to the 16-bit output dtype
                entry["floor_rounded_outputs"] = {
                    key: rel_l2(g.to(q.dtype), w) for key, g, w in zip(("dq", "dk", "dv"), got, want)
                }
        floors[name] = entry
    (HERE / "floor_large_logit.json").write_text(json.dumps(floors, indent=1) + "\n")
    print("wrote", HERE / "attention_fp64.npz", HERE / "floor_emulation.npz", HERE / "floor_large_logit.json")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/KohakuFA")
    main(sys.argv[1])
