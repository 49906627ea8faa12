"""The CPU oracle against the golden vectors produced by the reference's own code
(tests/golden/make_golden.py), plus internal consistency of the oracle and the workload recipes."""

from pathlib import Path

import numpy as np
import pytest
import torch

from kohakufa_b200 import workloads
from oracle import reference as oracle
from tests.golden import make_golden

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def attention_golden():
    return np.load(GOLDEN / "attention_fp64.npz")


@pytest.fixture(scope="module")
def floor_golden():
    return np.load(GOLDEN / "floor_emulation.npz")


@pytest.mark.parametrize("name", sorted(make_golden.ATTENTION_CASES))
def test_attention_fp64_matches_reference(name, attention_golden):
    case = make_golden.ATTENTION_CASES[name]
    q, k, v, dout = make_golden.make_attention_inputs(case)
    got = oracle.attention_fp64(q, k, v, dout, case[4] ** -0.5, block=case[6])
    for key, g in zip(("out", "dq", "dk", "dv"), got):
        want = torch.from_numpy(attention_golden[f"{name}/{key}"])
        # fp64 on both sides; only the order of summation differs (autograd vs explicit formulas)
        assert oracle.metrics(g, want)["rel_err"] < 1e-12, (name, key)
        assert float((g - want).abs().max()) < 1e-11, (name, key)


@pytest.mark.parametrize("name", sorted(make_golden.MASK_CASES))
def test_masked_and_grouped_attention_matches_reference(name, attention_golden):
    """Boolean masks (random, broadcast with empty rows, key padding) and grouped-query attention."""
    case = make_golden.MASK_CASES[name]
    q, k, v, dout, mask, block = make_golden.make_mask_inputs(case)
    got = oracle.attention_fp64(q, k, v, dout, case[5] ** -0.5, block=block, mask=mask, groups=case[1] // case[2])
    for key, g in zip(("out", "dq", "dk", "dv"), got):
        want = torch.from_numpy(attention_golden[f"{name}/{key}"])
        assert g.shape == want.shape, (name, key)
        assert bool(torch.isfinite(g).all()), (name, key)
        assert oracle.metrics(g, want)["rel_err"] < 1e-12, (name, key)
        assert float((g - want).abs().max()) < 1e-11, (name, key)


def test_rows_without_visible_keys_are_zero():
    case = make_golden.MASK_CASES["mask_broadcast_empty_rows_f16"]
    q, k, v, dout, mask, _ = make_golden.make_mask_inputs(case)
    out, dq, _, _ = oracle.attention_fp64(q, k, v, dout, case[5] ** -0.5, mask=mask)
    assert float(out[:, :, 5:10].abs().max()) == 0.0 and float(dq[:, :, 5:10].abs().max()) == 0.0


@pytest.mark.parametrize("name", sorted(make_golden.ATTENTION_CASES))
def test_metrics_match_reference(name, attention_golden):
    want_out = torch.from_numpy(attention_golden[f"{name}/out"])
    noisy = want_out + 1e-3 * torch.randn(
        want_out.shape, generator=torch.Generator().manual_seed(5), dtype=torch.float64
    )
    m = oracle.metrics(noisy, want_out)
    got = np.array([m["cos"], m["norm_ratio"], m["rel_err"], m["max_abs_err"], m["max_rel_err"]])
    np.testing.assert_allclose(got, attention_golden[f"{name}/metrics"], rtol=1e-12, atol=0)


@pytest.mark.parametrize("name", sorted(make_golden.FLOOR_CASES))
@pytest.mark.parametrize("tag", sorted(make_golden.BUG_SETS))
def test_floor_matches_reference(name, tag, floor_golden):
    case = make_golden.FLOOR_CASES[name]
    q, k, v, dout = make_golden.make_floor_inputs(case)
    got = oracle.floor_grads(q, k, v, dout, case[3] ** -0.5, bugs=frozenset(make_golden.BUG_SETS[tag]))
    for key, g in zip(("dq", "dk", "dv"), got):
        want = torch.from_numpy(floor_golden[f"{name}/{tag}/{key}"])
        assert torch.equal(g, want) or oracle.metrics(g, want)["rel_err"] < 1e-13, (name, tag, key)


def test_visible_rule():
    m = oracle.visible(5, 7, 2)
    want = torch.tensor([[c // 2 <= r // 2 for c in range(7)] for r in range(5)])
    assert torch.equal(m, want)
    assert oracle.visible(4, 4, 0) is None
    assert torch.equal(oracle.visible(3, 3, 1), torch.ones(3, 3).tril().bool())


def test_floor_is_close_to_fp64_and_bugs_are_worse():
    """On large-logit near-one-hot rows the floor stays near fp64 while each named bug does not:
    the 1.1x-floor bar of the parity tests discriminates."""
    cfg = workloads.CONFIGS["C2"]
    q, k, v, dout = workloads.make_inputs(cfg, batch=1, heads=2)
    want = oracle.attention_fp64(q, k, v, dout, cfg.scale)
    floor = oracle.floor_grads(q, k, v, dout, cfg.scale)
    floor_dk = oracle.rel_l2(floor[1], want[2])
    assert floor_dk < 5e-3
    for bug in ("single lse", "scale-shift"):
        bad = oracle.floor_grads(q, k, v, dout, cfg.scale, bugs=frozenset({bug}))
        assert oracle.rel_l2(bad[1], want[2]) > 1.5 * floor_dk, bug


@pytest.mark.parametrize("name", ["C2", "C2-bf16"])
def test_large_logit_recipe(name):
    cfg = workloads.CONFIGS[name]
    q, k, v, dout = workloads.make_inputs(cfg, batch=1, heads=2)
    s = (q.double() @ k.double().transpose(-1, -2)) * cfg.scale
    top = s.topk(2, dim=-1).values
    assert 0.8e5 < float(top[..., 0].median()) < 1.2e5
    gap = (top[..., 0] - top[..., 1])[..., : 2 * (cfg.seq // 2)]
    assert float(gap.median()) < 40.0
    assert torch.isfinite(k.float()).all()


def test_flop_convention():
    # causal S=8192: visible fraction (S + 1) / 2S
    f = workloads.attention_flops(4, 32, 8192, 8192, 128, block=1)
    assert abs(f / 7.698e12 - 1) < 1e-3
    f4 = workloads.attention_flops(8, 16, 4096, 4096, 64, block=256)
    assert abs(f4 / 1.0222e12 - 1) < 1e-3
    for sq, skv, blk in [(37, 50, 7), (64, 20, 5), (10, 10, 0), (9, 9, 1)]:
        assert workloads.attention_flops(1, 1, sq, skv, 8, blk) == oracle.attention_flops(1, 1, sq, skv, 8, blk)
        mask = oracle.visible(sq, skv, blk)
        pairs = sq * skv if mask is None else int(mask.sum())
        assert workloads.visible_pairs(sq, skv, blk) == pairs
