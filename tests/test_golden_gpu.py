"""The CUDA kernels against the committed golden vectors themselves: ``tests/golden/attention_fp64.npz``
holds what the reference's own fp64 function (KohakuFA tests/reference.py:15-34) returned for these seeded
inputs, so this comparison does not pass through this repository's restatement of the oracle at all."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from kohakufa_b200 import _lib, attention

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden  # noqa: E402

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    got, want = got.detach().double().cpu(), want.double()
    return float((got - want).norm() / want.norm().clamp_min(1e-300))


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN / "attention_fp64.npz")


def run_and_compare(name, golden, q, k, v, dout, tol, **kwargs):
    q, k, v = (t.cuda().requires_grad_() for t in (q, k, v))
    out = attention(q, k, v, **kwargs)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for key, g in zip(("out", "dq", "dk", "dv"), (out, q.grad, k.grad, v.grad)):
        want = torch.from_numpy(golden[f"{name}/{key}"])
        assert g.shape == want.shape, (name, key)
        if float(want.abs().max()) == 0.0:
            assert float(g.abs().max()) < 1e-4, (name, key)
        else:
            assert rel_err(g, want) < tol, (name, key, rel_err(g, want))


@pytest.mark.parametrize("name", sorted(make_golden.ATTENTION_CASES))
def test_kernels_match_reference_outputs(name, golden):
    case = make_golden.ATTENTION_CASES[name]
    q, k, v, dout = make_golden.make_attention_inputs(case)
    tol = 2e-2 if case[5] == "bfloat16" else 5e-3
    block = case[6]
    kwargs = {} if block == 0 else ({"causal": True} if block == 1 else {"block_causal": block})
    run_and_compare(name, golden, q, k, v, dout, tol, **kwargs)


@pytest.mark.parametrize("name", sorted(make_golden.MASK_CASES))
def test_masked_and_grouped_kernels_match_reference_outputs(name, golden):
    case = make_golden.MASK_CASES[name]
    q, k, v, dout, mask, block = make_golden.make_mask_inputs(case)
    tol = 2e-2 if case[6] == "bfloat16" else 5e-3
    if block == 1:
        kwargs = {"causal": True}
    else:  # like the reference's, attention() wants the mask's last two dimensions spelled out
        kwargs = {"mask": mask.expand(mask.shape[0], mask.shape[1], q.shape[2], k.shape[2]).cuda()}
    run_and_compare(name, golden, q, k, v, dout, tol, **kwargs)
