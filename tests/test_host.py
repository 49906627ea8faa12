"""CPU tests of the host side: argument handling of ``attention`` (same exceptions as the reference,
KohakuFA src/kohakufa/api.py:93-109 and sm100/op.py:41-55), the C-ABI library's exported symbols, and
the header / binding agreement. No kernel runs here."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

import kohakufa_b200
from kohakufa_b200 import _lib, api, op

ROOT = Path(__file__).resolve().parent.parent


def qkv(b=1, h=2, s=16, d=64, dtype=torch.float16):
    return tuple(torch.zeros(b, h, s, d, dtype=dtype) for _ in range(3))


def test_header_declares_what_the_binding_uses():
    header = (ROOT / "include" / "kfa.h").read_text()
    declared = set(re.findall(r"\b(kfa_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.SYMBOLS)


def test_library_exports_every_declared_symbol():
    from kohakufa_b200 import build

    path = build.build()
    lib = ctypes.CDLL(str(path))
    for name in _lib.SYMBOLS:
        assert hasattr(lib, name), name
    assert lib.kfa_abi_version() == _lib.ABI_VERSION
    lib.kfa_bwd_stats_bytes.restype = ctypes.c_int64
    lib.kfa_bwd_stats_bytes.argtypes = [ctypes.c_int64] * 3
    assert lib.kfa_bwd_stats_bytes(2, 3, 129) == 2 * 3 * 2 * 3 * 128 * 4


def test_library_rejects_bad_arguments_without_a_gpu():
    lib = _lib.load()
    t = _lib.KfaTensor4()
    t.ptr = 64
    for i, (n, s) in enumerate(zip((1, 2, 16, 40), (1280, 640, 40, 1))):  # head dim 40: not a multiple of 16
        t.shape[i], t.stride[i] = n, s
    rc = lib.kfa_fwd(ctypes.byref(t), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t), 64, 1.0, 0, 0, 64, None)
    assert rc == -1 and b"head_dim" in lib.kfa_last_error()
    t.shape[3] = 64
    t.stride[2] = 60
    rc = lib.kfa_fwd(ctypes.byref(t), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t), 64, 1.0, 0, 0, 64, None)
    assert rc == -1 and b"stride" in lib.kfa_last_error()


def test_causal_and_block_causal_are_exclusive():
    q, k, v = qkv()
    with pytest.raises(ValueError, match="causal is block_causal=1"):
        api.attention(q, k, v, causal=True, block_causal=4)


def test_compute_dtype_must_be_16_bit():
    q, k, v = qkv()
    with pytest.raises(TypeError, match="compute_dtype"):
        api.attention(q, k, v, compute_dtype=torch.float32)


def test_head_dim_range():
    q, k, v = qkv(d=136)
    with pytest.raises(ValueError, match="head_dim 136"):
        api.attention(q, k, v)


def test_mask_with_block_rejected_first():
    q, k, v = qkv()
    with pytest.raises(ValueError, match="mask or causal"):
        api.attention(q, k, v, causal=True, mask=torch.ones(16, 16, dtype=torch.bool))
    with pytest.raises(ValueError, match="CUDA tensors only"):  # masks are built; CPU tensors are not
        api.attention(q, k, v, mask=torch.ones(16, 16, dtype=torch.bool))


def test_check_rules():
    q, k, v = qkv()
    with pytest.raises(TypeError):
        op._check(q.float(), k.float(), v.float())
    with pytest.raises(TypeError):
        op._check(q, k.bfloat16(), v)
    with pytest.raises(ValueError, match="k .* vs q"):
        op._check(q, k, v[:, :, :8])
    with pytest.raises(ValueError, match="multiple of K / V heads"):
        op._check(torch.zeros(1, 3, 16, 64, dtype=torch.float16), k, v)
    with pytest.raises(ValueError, match="CUDA tensors only"):
        op._check(q, k, v)
    with pytest.raises(ValueError, match="head_dim"):
        op._check(*qkv(d=40))  # the op takes multiples of 16; api.attention pads other head dims


def test_stride_rule():
    x = torch.zeros(1, 2, 16, 72, dtype=torch.float16)
    assert op._strides_ok(x)
    assert not op._strides_ok(x.transpose(-1, -2))  # last dim not contiguous
    assert not op._strides_ok(torch.zeros(1, 2, 16, 68, dtype=torch.float16)[..., :64])  # 136-byte rows
    assert not op._strides_ok(torch.zeros(1, 1, 1, 64, dtype=torch.float16).expand(1, 2, 16, 64))


def test_pad_head_dim():
    q, k, v = qkv(d=40)
    pq, pk, pv = api._fit_head_dim(q, k, v)
    assert pq.shape[-1] == pk.shape[-1] == pv.shape[-1] == 48  # the next multiple of 16 (reference api.py:18-29)
    assert torch.equal(pq[..., :40], q) and float(pq[..., 40:].abs().max()) == 0.0
    q, k, v = qkv(d=72)
    assert api._fit_head_dim(q, k, v)[0].shape[-1] == 80
    for d in (16, 96, 128):
        q, k, v = qkv(d=d)
        assert api._fit_head_dim(q, k, v)[0] is q


def test_center_keys_is_a_pure_shift():
    k = torch.randn(2, 3, 10, 8)
    c = api._remove_key_mean(k, torch.float16)
    assert c.dtype == torch.float16
    assert float(c.float().mean(-2).abs().max()) < 1e-3


def test_other_exports_raise():
    reference_exports = {"PackedMask", "attention", "attention_varlen", "pack_mask", "varlen_plan"}
    own = {"check_status", "reset_status", "set_deterministic", "is_deterministic", "set_backward", "get_backward"}
    assert set(kohakufa_b200.__all__) == reference_exports | own


def test_mask_normalize_rules():
    from kohakufa_b200 import mask

    with pytest.raises(TypeError):
        mask.normalize(torch.ones(3, 3), 1, 1, 3, 3)
    with pytest.raises(ValueError):
        mask.normalize(torch.ones(3, 4, dtype=torch.bool), 1, 1, 3, 3)
    with pytest.raises(ValueError):
        mask.normalize(torch.ones(2, 1, 3, 3, dtype=torch.bool), 3, 1, 3, 3)
    assert mask.normalize(torch.ones(3, 3, dtype=torch.bool), 2, 2, 3, 3).shape == (1, 1, 3, 3)
    assert mask.words_per_row(1) == 4 and mask.words_per_row(128) == 4 and mask.words_per_row(129) == 8
    with pytest.raises(ValueError, match="CUDA"):
        kohakufa_b200.pack_mask(torch.ones(3, 3, dtype=torch.bool), 1, 1, 3, 3)


def test_varlen_plan_reads_lengths_once_and_validates():
    cu_q = torch.tensor([0, 5, 5, 300], dtype=torch.int32)
    cu_k = torch.tensor([0, 9, 9, 100], dtype=torch.int32)
    assert kohakufa_b200.varlen_plan(cu_q, cu_k, 4, 2, 1) == (3, 295, 91)
    with pytest.raises(ValueError):  # queries without keys
        kohakufa_b200.varlen_plan(cu_q, torch.tensor([0, 9, 100, 100], dtype=torch.int32))
    with pytest.raises(ValueError):  # different numbers of sequences
        kohakufa_b200.varlen_plan(cu_q, cu_k[:-1])
    with pytest.raises(ValueError):  # decreasing
        kohakufa_b200.varlen_plan(torch.tensor([0, 9, 5], dtype=torch.int32), torch.tensor([0, 9, 12], dtype=torch.int32))


def test_varlen_fake_kernels_infer_layouts():
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        q = torch.empty(300, 4, 64, dtype=torch.float16, device="cuda")
        k = torch.empty(100, 2, 64, dtype=torch.float16, device="cuda")
        cu = torch.empty(4, dtype=torch.int32, device="cuda")
        out, lse = torch.ops.kohakufa_b200.sm100_varlen_forward(q, k, k, cu, cu, 295, 91, 0.125, 1)
        assert out.shape == q.shape and lse.shape == (1, 4, 2, 300) and lse.dtype == torch.float32
        dq, dk, dv = torch.ops.kohakufa_b200.sm100_varlen_backward(q, k, k, out, out, lse, cu, cu, 295, 91, 0.125, 1)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == k.shape


def test_center_keys_varlen_subtracts_each_sequence_mean():
    from kohakufa_b200.api import _remove_key_mean

    k = torch.randn(12, 2, 8) + 3.0
    cu = torch.tensor([0, 5, 5, 12], dtype=torch.int32)
    c = _remove_key_mean(k, k.dtype, cu)
    assert float(c[:5].mean(0).abs().max()) < 1e-5 and float(c[5:].mean(0).abs().max()) < 1e-5


def test_fake_kernels_infer_layouts():
    """The registered fakes give the [B, S, H, D]-storage views without touching a device."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        q = torch.empty(2, 10, 3, 64, dtype=torch.float16, device="cuda").transpose(1, 2)
        k = torch.empty(2, 14, 3, 64, dtype=torch.float16, device="cuda").transpose(1, 2)
        out, lse = torch.ops.kohakufa_b200.sm100_forward(q, k, k, 0.125, 0)
        assert out.shape == (2, 3, 10, 64) and out.stride() == (10 * 3 * 64, 64, 3 * 64, 1)
        assert lse.shape == (2, 3, 2, 10) and lse.dtype == torch.float32
        dq, dk, dv = torch.ops.kohakufa_b200.sm100_backward(q, k, k, out, out, lse, 0.125, 0)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.stride() == k.stride()


def test_bench_clock_sampler_with_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """ClockSampler parses nvidia-smi rows, keeps only the rows sampled after wait_running(), and reports
    throttle reasons; nvidia-smi is replaced by a script that prints rows like the real one."""
    import importlib
    import os
    import stat
    import time

    fake = tmp_path / "nvidia-smi"
    fake.write_text(
        "#!/bin/sh\n"
        "echo '1965, 1965, 150.0, Not Active, Not Active, Not Active, Not Active'\n"
        "sleep 0.3\n"
        "while true; do echo '1700, 1965, 990.0, Not Active, Not Active, Not Active, Active'; sleep 0.05; done\n"
    )
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    bench = importlib.import_module("bench")
    with bench.ClockSampler(0) as sampler:
        sampler.wait_running()
        assert sampler.first == 1  # the idle row came before the timed region
        t0 = time.perf_counter()
        while sampler.samples_under_load() < 3 and time.perf_counter() - t0 < 5:
            time.sleep(0.05)
    out = sampler.summary()
    assert out["sm_mhz"] == 1700.0 and out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"]
    assert out["samples"] >= 3
    assert bench.ClockSampler(-1).summary()["samples"] == 0


def test_bench_notes():
    import importlib

    bench = importlib.import_module("bench")
    from kohakufa_b200 import workloads

    assert "larger than L2" in bench.l2_note(workloads.CONFIGS["C3"])
    assert "fit in L2" in bench.l2_note(workloads.CONFIGS["C1"])
    assert set(bench.PUBLISHED) == {"C4"}
    d = bench.config_dict(workloads.CONFIGS["C5"], 8)
    assert "ring over 8 GPUs" in d["parallelism"] and d["global_batch"] == 1
