"""ctypes binding of ``libkfa.so`` (declared in ``include/kfa.h``).

The library is the only compute path of this package: there is no Python, Triton or CPU
fallback. If it is missing, loading raises with the build command instead of degrading.
"""

import ctypes
import threading
from pathlib import Path

import torch

import os

# The in-tree build; the environment variable KFA_LIBRARY points the package at another build of the same
# sources (e.g. one compiled with different tuning macros) without touching the tree.
LIB_PATH = Path(os.environ.get("KFA_LIBRARY") or Path(__file__).resolve().parent / "libkfa.so")

KFA_F16, KFA_BF16 = 0, 1
ABI_VERSION = 1

# Every entry point include/kfa.h declares (checked against the built library by the tests).
SYMBOLS = (
    "kfa_abi_version",
    "kfa_last_error",
    "kfa_bwd_stats_bytes",
    "kfa_fwd",
    "kfa_bwd_prepare",
    "kfa_bwd_dkdv",
    "kfa_bwd_dq",
    "kfa_bwd",
    "kfa_bwd_dq_acc_bytes",
    "kfa_bwd_prepare_fused",
    "kfa_bwd_fused_main",
    "kfa_bwd_dq_convert",
    "kfa_bwd_fused",
    "kfa_bwd_static_scratch",
    "kfa_fwd_varlen",
    "kfa_bwd_varlen",
    "kfa_pack_mask",
    "kfa_fwd_masked",
    "kfa_bwd_masked",
    "kfa_cp_fwd_step",
    "kfa_cp_fwd_finalize",
    "kfa_cp_bwd_dkdv_step",
    "kfa_cp_bwd_dq_step",
    "kfa_cp_grad_finalize",
    "kfa_copy_rows",
    "kfa_scores",
    "kfa_selftest",
)


class KfaTensor4(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("shape", ctypes.c_int64 * 4),
        ("stride", ctypes.c_int64 * 4),
    ]


class KfaMaskWords(ctypes.Structure):
    _fields_ = [
        ("words", ctypes.c_void_p),
        ("stride_batch", ctypes.c_int64),
        ("stride_head", ctypes.c_int64),
        ("stride_row", ctypes.c_int64),
    ]


class KfaMaskTiles(ctypes.Structure):
    _fields_ = [("any", ctypes.c_void_p), ("stride_batch", ctypes.c_int64), ("stride_head", ctypes.c_int64)]


class KfaAcc32(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("head_stride", ctypes.c_int64)]


def acc32(t: torch.Tensor, row0: int = 0) -> KfaAcc32:
    """Descriptor of a contiguous fp32 ``[B, H, S, D]`` accumulator, optionally starting at row ``row0``."""
    assert t.dtype == torch.float32 and t.is_contiguous() and t.dim() == 4
    a = KfaAcc32()
    a.ptr = t.data_ptr() + 4 * row0 * t.shape[3]
    a.head_stride = t.shape[2] * t.shape[3]
    return a


class KfaError(RuntimeError):
    """A libkfa call returned a negative status."""


_lock = threading.Lock()
_lib = None
_status = {}  # device index -> int32[1] status word


def load() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise KfaError(
                f"{LIB_PATH} is missing: build it with `python -m kohakufa_b200.build` "
                "(needs nvcc; there is no fallback path)"
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        T = ctypes.POINTER(KfaTensor4)
        vp, fp, ip = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p
        lib.kfa_abi_version.restype = ctypes.c_int
        lib.kfa_last_error.restype = ctypes.c_char_p
        lib.kfa_bwd_stats_bytes.restype = ctypes.c_int64
        lib.kfa_bwd_stats_bytes.argtypes = [ctypes.c_int64] * 3
        lib.kfa_fwd.argtypes = [T, T, T, T, fp, ctypes.c_float, ctypes.c_int, ctypes.c_int, ip, vp]
        lib.kfa_bwd_prepare.argtypes = [T, T, fp, fp, ctypes.c_int, vp]
        lib.kfa_bwd_dkdv.argtypes = [T, T, T, T, fp, T, T, ctypes.c_float, ctypes.c_int, ctypes.c_int, ip, vp]
        lib.kfa_bwd_dq.argtypes = [T, T, T, T, fp, T, ctypes.c_float, ctypes.c_int, ctypes.c_int, ip, vp]
        lib.kfa_bwd.argtypes = [T, T, T, T, T, fp, fp, T, T, T, ctypes.c_float, ctypes.c_int, ctypes.c_int, ip, vp]
        lib.kfa_bwd_dq_acc_bytes.restype = ctypes.c_int64
        lib.kfa_bwd_dq_acc_bytes.argtypes = [ctypes.c_int64] * 4
        lib.kfa_bwd_prepare_fused.argtypes = [T, T, fp, fp, fp, ctypes.c_int, vp]
        lib.kfa_bwd_fused_main.argtypes = [T, T, T, T, fp, fp, T, T, ctypes.c_float, ctypes.c_int, ctypes.c_int, ip, vp]
        lib.kfa_bwd_dq_convert.argtypes = [fp, T, ctypes.c_float, ctypes.c_int, ip, vp]
        lib.kfa_bwd_fused.argtypes = [T, T, T, T, T, fp, fp, fp, T, T, T, ctypes.c_float, ctypes.c_int, ctypes.c_int, ip, vp]
        lib.kfa_bwd_static_scratch.argtypes = [T, T, T, T, T, fp, T, T, T, ctypes.c_float, ctypes.c_int, ctypes.c_int, ip, vp]
        A = ctypes.POINTER(KfaAcc32)
        i64, f32, i32 = ctypes.c_int64, ctypes.c_float, ctypes.c_int
        M = ctypes.POINTER(KfaMaskWords)
        MT = ctypes.POINTER(KfaMaskTiles)
        lib.kfa_pack_mask.argtypes = [vp, ctypes.POINTER(ctypes.c_int64), i32, i32, i32, i32, ip, ip, ip, vp]
        lib.kfa_fwd_masked.argtypes = [T, T, T, T, fp, M, MT, f32, i32, ip, vp]
        lib.kfa_bwd_masked.argtypes = [T, T, T, T, T, fp, fp, T, T, T, M, M, MT, f32, i32, ip, vp]
        lib.kfa_fwd_varlen.argtypes = [T, T, T, T, fp, ip, ip, i32, i32, i32, f32, i32, i32, ip, vp]
        lib.kfa_bwd_varlen.argtypes = [T, T, T, T, T, fp, fp, T, T, T, ip, ip, i32, i32, i32, f32, i32, i32, ip, vp]
        lib.kfa_cp_fwd_step.argtypes = [T, T, T, A, fp, i64, i64, i32, f32, i32, i32, ip, vp]
        lib.kfa_cp_fwd_finalize.argtypes = [A, fp, i64, i64, T, fp, i32, vp]
        lib.kfa_cp_bwd_dkdv_step.argtypes = [T, T, T, T, fp, i64, A, A, i32, f32, i32, i32, ip, vp]
        lib.kfa_cp_bwd_dq_step.argtypes = [T, T, T, T, fp, i64, A, i32, f32, i32, i32, ip, vp]
        lib.kfa_cp_grad_finalize.argtypes = [A, T, i32, vp]
        lib.kfa_copy_rows.argtypes = [vp, i64, vp, i64, i64, i64, i32, vp]
        lib.kfa_scores.argtypes = [T, T, fp, i32, ip, vp]
        lib.kfa_selftest.argtypes = [ctypes.c_char_p, ctypes.c_int]
        for name in SYMBOLS:
            if name not in ("kfa_abi_version", "kfa_last_error", "kfa_bwd_stats_bytes", "kfa_bwd_dq_acc_bytes"):
                getattr(lib, name).restype = ctypes.c_int
        if lib.kfa_abi_version() != ABI_VERSION:
            raise KfaError(f"libkfa ABI {lib.kfa_abi_version()} != expected {ABI_VERSION}: rebuild")
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise KfaError(f"libkfa error {rc}: {load().kfa_last_error().decode()}")


def tensor4(t: torch.Tensor) -> KfaTensor4:
    """Descriptor of a [B, H, S, D] CUDA tensor (any strides; validated by the library)."""
    assert t.dim() == 4 and t.is_cuda
    d = KfaTensor4()
    d.ptr = t.data_ptr()
    for i in range(4):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    return d


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return KFA_F16
    if dtype == torch.bfloat16:
        return KFA_BF16
    raise TypeError(f"libkfa: dtype {dtype}: fp16 or bf16")


def status_word(device: torch.device) -> torch.Tensor:
    """The per-device int32 word kernels report a timed-out wait in (0 = healthy)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _status.get(index)
    if word is None:
        with _lock:
            word = _status.get(index)
            if word is None:
                word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
                _status[index] = word
    return word


def device_status(device=None) -> int:
    """Reads the status word back (synchronises). Nonzero: 100 + id of the wait that gave up."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(status_word(device).item())


def reset_device_status(device=None) -> None:
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    status_word(device).zero_()


def check_status(device=None) -> None:
    """Raises ``KfaError`` if a kernel on ``device`` (default: the current one) gave up on an internal
    wait since the last ``reset_status``.

    The kernels never hang: a wait that exceeds its (seconds-long) limit makes the CTA fill the output
    rows it owns with NaN, record ``100 + wait id`` in a per-device status word and leave; every later
    launch on that device then skips its work and leaves its outputs as NaN as well. Nothing on the
    launch path reads the word back (that would synchronise), so call this where the program
    synchronises anyway, e.g. after ``loss.item()`` or the optimizer step: NaN gradients plus a nonzero
    status mean "a kernel timed out", not "the model diverged". Reads one int from the device."""
    code = device_status(device)
    if code != 0:
        raise KfaError(
            f"a libkfa kernel timed out waiting on its pipeline (status {code} = 100 + wait id); outputs since then "
            "are NaN. Call reset_status() to re-enable the kernels"
        )


def reset_status(device=None) -> None:
    """Clears the device's status word (see ``check_status``) so that later launches do their work again."""
    reset_device_status(device)


def raw_scores(q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """``q k^T`` (unscaled, unmasked) as fp32 ``[B, H, Sq, Skv]``, straight from the tensor-core instruction
    sequence the attention kernels use (``kfa_scores``): a diagnostic for accuracy studies."""
    out = torch.empty(q.shape[0], q.shape[1], q.shape[2], k.shape[2], dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        rc = load().kfa_scores(
            ctypes.byref(tensor4(q)),
            ctypes.byref(tensor4(k)),
            out.data_ptr(),
            dtype_code(q.dtype),
            status_word(q.device).data_ptr(),
            stream_ptr(q.device),
        )
    check(rc)
    return out


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def selftest() -> str:
    """Runs the library's hardware self-check on the current device; returns its report."""
    buf = ctypes.create_string_buffer(4096)
    rc = load().kfa_selftest(buf, len(buf))
    report = buf.value.decode()
    if rc != 0:
        raise KfaError(f"kfa_selftest failed ({rc}): {load().kfa_last_error().decode()}\n{report}")
    return report
