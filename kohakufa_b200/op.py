"""The sm_100a kernels as torch custom ops with autograd: ``attention(q, k, v, scale, block_causal)``.

Mirrors the operator boundary of the reference (KohakuFA ``src/kohakufa/sm100/op.py:41-175``):

    q [B, H, Sq, D], k / v [B, H, Skv, D], fp16 or bf16 (views of [B, S, H, D] projections are
    fine: any strides with a contiguous last dim and 16-byte aligned strides), D a multiple of 16 up to 128.
    scale: softmax scale (None -> D ** -0.5). block_causal: frame size P (query i sees key j iff
    j // P <= i // P), 0 for dense attention.
    Returns out [B, H, Sq, D], a view of [B, Sq, H, D] storage.

The ops live in their own namespace (``kohakufa_b200::sm100_forward`` / ``_backward``; the
reference registers ``kohakufa::sm100_*``), so both packages can be imported side by side.
Their bodies call ``libkfa.so`` through ctypes on the current stream: no host synchronisation,
every buffer from the caching allocator, so ``torch.compile`` keeps them in the graph and CUDA
graph capture works (after one eager call on the device, which creates the status word).

Extra memory: forward statistics (row max and log2 sum, fp32 [B, H, 2, Sq]); backward
(m, log2 l, delta) per query row (fp32, padded to 128 rows) while it runs.
"""

import ctypes

import torch
from torch import Tensor

from kohakufa_b200 import _lib

import os

KERNEL_DIMS = tuple(range(16, 129, 16))  # head dims the kernels are built for (the reference's multiples of 16: api.py:18-29); the API zero-pads up to one
FUSED_DIMS = (64, 128)  # ... and those the fused backward is built for
MAX_KERNEL_DIM = 128


def kernel_dim_for(dim: int) -> int:
    """The smallest head dim a kernel is built for that holds ``dim``."""
    return min(d for d in KERNEL_DIMS if d >= dim)


# Which backward runs. Two implementations exist:
#   fused  one key-major kernel, dK, dV and dQ from one P and one dS per tile pair (five matrix products),
#          dQ accumulated across key tiles with fp32 reduce-adds in global memory: its last bits vary from
#          run to run with the order of those adds;
#   split  a dK / dV kernel plus a dQ kernel that recomputes S and dP (seven matrix products): bit-identical
#          gradients every run.
# "auto" picks by measured speed on B200: at head dim 64 the fused kernel wins (the backward is bound by the
# exponentials, which it computes once); at head dim 128 the reduce-add traffic (64 KB per tile pair into
# L2) costs more than the two recomputed products, and the split kernels win.
_backward_mode = os.environ.get("KFA_BACKWARD", "auto")
if os.environ.get("KFA_DETERMINISTIC", "0") not in ("", "0"):
    _backward_mode = "split"
FUSED_IS_FASTER = {64: True, 128: False}


def set_backward(mode: str) -> None:
    """``"auto"`` (default), ``"fused"`` or ``"split"``: the backward implementation of dense / causal /
    block-causal ``attention`` (masks and packed batches always run the split kernels). Also settable with
    the environment variable ``KFA_BACKWARD`` before the import."""
    global _backward_mode
    if mode not in ("auto", "fused", "split"):
        raise ValueError(f"backward mode {mode!r}: 'auto', 'fused' or 'split'")
    _backward_mode = mode


def get_backward() -> str:
    return _backward_mode


def set_deterministic(flag: bool) -> None:
    """``True``: every later backward uses the split kernels, whose gradients repeat bit for bit;
    ``False``: back to ``"auto"``. (``KFA_DETERMINISTIC=1`` in the environment does the same.)"""
    set_backward("split" if flag else "auto")


def is_deterministic() -> bool:
    return _backward_mode == "split"


def use_fused_backward(dim: int, batch_heads: int) -> bool:
    """Whether the fused kernel runs for this head dim under the current mode."""
    if _backward_mode == "split" or batch_heads > 65535:
        return False
    if dim not in FUSED_DIMS:
        return False
    return _backward_mode == "fused" or FUSED_IS_FASTER[dim]


def _strides_ok(t: Tensor) -> bool:
    if t.stride(-1) != 1:  # (the base address is checked by the library: 16-byte aligned)
        return False
    return all(s > 0 and (s * 2) % 16 == 0 for n, s in zip(t.shape[:-1], t.stride()[:-1]) if n > 1)


def _check(q: Tensor, k: Tensor, v: Tensor) -> None:
    """Same conditions and exception types as the reference's ``_check`` (op.py:41-55), with the
    head dims and head counts this library supports."""
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("attention: q, k, v must be fp16 or bf16 (all the same)")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("attention: q, k, v must be [B, H, S, D]")
    dim = q.shape[-1]
    if dim not in KERNEL_DIMS:
        raise ValueError(f"attention: kernel head_dim {dim}: one of {KERNEL_DIMS}")
    if k.shape != v.shape or k.shape[0] != q.shape[0] or k.shape[-1] != q.shape[-1]:
        raise ValueError(f"attention: k {tuple(k.shape)} / v {tuple(v.shape)} vs q {tuple(q.shape)}")
    if q.shape[1] % k.shape[1]:
        raise ValueError("attention: query heads must be a multiple of K / V heads (GQA)")
    if not q.is_cuda:
        raise ValueError("attention: CUDA tensors only (there is no CPU path)")
    for t in (q, k, v):
        if not _strides_ok(t):
            raise ValueError("attention: inputs need a contiguous last dim and 16-byte strides")


def _bshd_like(t: Tensor) -> Tensor:
    batch, heads, seq, dim = t.shape
    return t.new_empty(batch, seq, heads, dim).transpose(1, 2)


@torch.library.custom_op("kohakufa_b200::sm100_forward", mutates_args=(), device_types="cuda")
def attention_fwd_op(q: Tensor, k: Tensor, v: Tensor, scale: float, block: int) -> tuple[Tensor, Tensor]:
    lib = _lib.load()
    batch, heads, seq_q, _ = q.shape
    out = _bshd_like(q)
    lse = q.new_empty(batch, heads, 2, seq_q, dtype=torch.float32)
    with torch.cuda.device(q.device):
        rc = lib.kfa_fwd(
            ctypes.byref(_lib.tensor4(q)),
            ctypes.byref(_lib.tensor4(k)),
            ctypes.byref(_lib.tensor4(v)),
            ctypes.byref(_lib.tensor4(out)),
            lse.data_ptr(),
            float(scale),
            int(block),
            _lib.dtype_code(q.dtype),
            _lib.status_word(q.device).data_ptr(),
            _lib.stream_ptr(q.device),
        )
    _lib.check(rc)
    return out, lse


@attention_fwd_op.register_fake
def _(q, k, v, scale, block):
    batch, heads, seq_q, dim = q.shape
    out = q.new_empty(batch, seq_q, heads, dim).transpose(1, 2)
    lse = q.new_empty(batch, heads, 2, seq_q, dtype=torch.float32)
    return out, lse


@torch.library.custom_op("kohakufa_b200::sm100_backward", mutates_args=(), device_types="cuda")
def attention_bwd_op(
    q: Tensor, k: Tensor, v: Tensor, out: Tensor, dout: Tensor, lse: Tensor, scale: float, block: int
) -> tuple[Tensor, Tensor, Tensor]:
    lib = _lib.load()
    batch, heads, seq_q, dim = q.shape
    dq, dk, dv = _bshd_like(q), _bshd_like(k), _bshd_like(v)
    stats = q.new_empty(lib.kfa_bwd_stats_bytes(batch, heads, seq_q) // 4, dtype=torch.float32)
    tensors = [ctypes.byref(_lib.tensor4(t)) for t in (q, k, v, out, dout, dq, dk, dv)]
    tail = (
        float(scale),
        int(block),
        _lib.dtype_code(q.dtype),
        _lib.status_word(q.device).data_ptr(),
        _lib.stream_ptr(q.device),
    )
    with torch.cuda.device(q.device):
        if not use_fused_backward(dim, batch * heads):
            rc = lib.kfa_bwd(*tensors[:5], lse.data_ptr(), stats.data_ptr(), *tensors[5:], *tail)
        else:
            dq_acc = q.new_empty(lib.kfa_bwd_dq_acc_bytes(batch, heads, seq_q, dim) // 4, dtype=torch.float32)
            rc = lib.kfa_bwd_fused(
                *tensors[:5], lse.data_ptr(), stats.data_ptr(), dq_acc.data_ptr(), *tensors[5:], *tail
            )
    _lib.check(rc)
    return dq, dk, dv


@attention_bwd_op.register_fake
def _(q, k, v, out, dout, lse, scale, block):
    return _bshd_like(q), _bshd_like(k), _bshd_like(v)


def _setup_context(ctx, inputs, output):
    q, k, v, scale, block = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse)
    ctx.scale = scale
    ctx.block = block
    ctx.mark_non_differentiable(lse)


def _backward(ctx, dout, dlse):
    q, k, v, out, lse = ctx.saved_tensors
    if not _strides_ok(dout):  # e.g. an expanded gradient: same rule as the reference (op.py:135-136)
        dout = dout.contiguous()
    dq, dk, dv = attention_bwd_op(q, k, v, out, dout, lse, ctx.scale, ctx.block)
    return dq, dk, dv, None, None


attention_fwd_op.register_autograd(_backward, setup_context=_setup_context)


# --------------------------------------------------------------------------------------
# Boolean masks: ops of their own (the reference passes optional word tensors to its one op pair,
# op.py:58-121); the packed words are saved for the backward.
# --------------------------------------------------------------------------------------


@torch.library.custom_op("kohakufa_b200::sm100_masked_forward", mutates_args=(), device_types="cuda")
def masked_fwd_op(
    q: Tensor, k: Tensor, v: Tensor, words: Tensor, words_t: Tensor, tiles: Tensor, scale: float
) -> tuple[Tensor, Tensor]:
    from kohakufa_b200.mask import mask_tiles, mask_words

    lib = _lib.load()
    batch, heads, seq_q, _ = q.shape
    out = _bshd_like(q)
    lse = q.new_empty(batch, heads, 2, seq_q, dtype=torch.float32)
    with torch.cuda.device(q.device):
        rc = lib.kfa_fwd_masked(
            *(ctypes.byref(_lib.tensor4(t)) for t in (q, k, v, out)),
            lse.data_ptr(),
            ctypes.byref(mask_words(words, batch, heads)),
            ctypes.byref(mask_tiles(tiles)),
            float(scale),
            _lib.dtype_code(q.dtype),
            _lib.status_word(q.device).data_ptr(),
            _lib.stream_ptr(q.device),
        )
    _lib.check(rc)
    return out, lse


@masked_fwd_op.register_fake
def _(q, k, v, words, words_t, tiles, scale):
    batch, heads, seq_q, dim = q.shape
    return q.new_empty(batch, seq_q, heads, dim).transpose(1, 2), q.new_empty(batch, heads, 2, seq_q, dtype=torch.float32)


@torch.library.custom_op("kohakufa_b200::sm100_masked_backward", mutates_args=(), device_types="cuda")
def masked_bwd_op(
    q: Tensor, k: Tensor, v: Tensor, out: Tensor, dout: Tensor, lse: Tensor, words: Tensor, words_t: Tensor,
    tiles: Tensor, scale: float,
) -> tuple[Tensor, Tensor, Tensor]:  # fmt: skip
    from kohakufa_b200.mask import mask_tiles, mask_words

    lib = _lib.load()
    batch, heads, seq_q, _ = q.shape
    dq, dk, dv = _bshd_like(q), _bshd_like(k), _bshd_like(v)
    stats = q.new_empty(lib.kfa_bwd_stats_bytes(batch, heads, seq_q) // 4, dtype=torch.float32)
    with torch.cuda.device(q.device):
        rc = lib.kfa_bwd_masked(
            *(ctypes.byref(_lib.tensor4(t)) for t in (q, k, v, out, dout)),
            lse.data_ptr(),
            stats.data_ptr(),
            *(ctypes.byref(_lib.tensor4(t)) for t in (dq, dk, dv)),
            ctypes.byref(mask_words(words, batch, heads)),
            ctypes.byref(mask_words(words_t, batch, heads)),
            ctypes.byref(mask_tiles(tiles)),
            float(scale),
            _lib.dtype_code(q.dtype),
            _lib.status_word(q.device).data_ptr(),
            _lib.stream_ptr(q.device),
        )
    _lib.check(rc)
    return dq, dk, dv


@masked_bwd_op.register_fake
def _(q, k, v, out, dout, lse, words, words_t, tiles, scale):
    return _bshd_like(q), _bshd_like(k), _bshd_like(v)


def _masked_setup(ctx, inputs, output):
    q, k, v, words, words_t, tiles, scale = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse, words, words_t, tiles)
    ctx.scale = scale
    ctx.mark_non_differentiable(lse)


def _masked_backward(ctx, dout, dlse):
    q, k, v, out, lse, words, words_t, tiles = ctx.saved_tensors
    if not _strides_ok(dout):
        dout = dout.contiguous()
    dq, dk, dv = masked_bwd_op(q, k, v, out, dout, lse, words, words_t, tiles, ctx.scale)
    return dq, dk, dv, None, None, None, None


masked_fwd_op.register_autograd(_masked_backward, setup_context=_masked_setup)


def attention(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    scale: float | None = None,
    block_causal: int = 0,
    mask=None,
) -> Tensor:
    """``softmax(scale q k^T) v`` over ``[B, H, S, D]``; ``block_causal > 0``: tokens of block ``i``
    (``block_causal`` consecutive tokens) see blocks ``0..i`` only; ``mask``: a bool mask broadcastable
    to ``[B, H, Sq, Skv]`` (True = visible; a row with no visible key outputs 0) or a ``PackedMask``
    (reference: op.py:146-175)."""
    from kohakufa_b200.mask import PackedMask

    _check(q, k, v)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    if mask is not None:
        if block_causal:
            raise ValueError("attention: give a mask or block_causal, not both (fold it in)")
        shape = (q.shape[0], q.shape[1], q.shape[2], k.shape[2])
        packed = mask if isinstance(mask, PackedMask) else PackedMask(mask, *shape)
        if packed.shape != shape:
            raise ValueError(f"packed mask for {packed.shape}, inputs are {shape}")
        out, _ = masked_fwd_op(q, k, v, packed.words, packed.words_t, packed.tiles, float(scale))
        return out
    out, _ = attention_fwd_op(q, k, v, float(scale), int(block_causal))
    return out


# --------------------------------------------------------------------------------------
# Variable-length (packed) sequences. Mirrors the reference's varlen ops (op.py:183-289); the plan is
# three host integers instead of device tile tables, because the kernels read the sequence
# boundaries themselves and return at once for tiles past a sequence's end.
# --------------------------------------------------------------------------------------


def _as4(t: Tensor) -> Tensor:
    """``[T, H, D]`` packed tensor as the ``[1, H, T, D]`` view the library takes."""
    return t.unsqueeze(0).transpose(1, 2)


@torch.library.custom_op("kohakufa_b200::sm100_varlen_forward", mutates_args=(), device_types="cuda")
def varlen_fwd_op(
    q: Tensor, k: Tensor, v: Tensor, cu_seqlens_q: Tensor, cu_seqlens_k: Tensor, max_q: int, max_k: int,
    scale: float, block: int,
) -> tuple[Tensor, Tensor]:  # fmt: skip
    lib = _lib.load()
    total_q, heads, _ = q.shape
    # zero-filled: rows no CTA writes (a sequence with queries but no keys, rows outside cu_seqlens) read
    # as "no visible key": output 0, statistics 0
    out = torch.zeros_like(q)
    lse = q.new_zeros(1, heads, 2, total_q, dtype=torch.float32)
    with torch.cuda.device(q.device):
        rc = lib.kfa_fwd_varlen(
            *(ctypes.byref(_lib.tensor4(_as4(t))) for t in (q, k, v, out)),
            lse.data_ptr(),
            cu_seqlens_q.data_ptr(),
            cu_seqlens_k.data_ptr(),
            cu_seqlens_q.numel() - 1,
            max_q,
            max_k,
            float(scale),
            int(block),
            _lib.dtype_code(q.dtype),
            _lib.status_word(q.device).data_ptr(),
            _lib.stream_ptr(q.device),
        )
    _lib.check(rc)
    return out, lse


@varlen_fwd_op.register_fake
def _(q, k, v, cu_seqlens_q, cu_seqlens_k, max_q, max_k, scale, block):
    return torch.empty_like(q), q.new_empty(1, q.shape[1], 2, q.shape[0], dtype=torch.float32)


@torch.library.custom_op("kohakufa_b200::sm100_varlen_backward", mutates_args=(), device_types="cuda")
def varlen_bwd_op(
    q: Tensor, k: Tensor, v: Tensor, out: Tensor, dout: Tensor, lse: Tensor, cu_seqlens_q: Tensor,
    cu_seqlens_k: Tensor, max_q: int, max_k: int, scale: float, block: int,
) -> tuple[Tensor, Tensor, Tensor]:  # fmt: skip
    lib = _lib.load()
    n_seqs = cu_seqlens_q.numel() - 1
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)  # unwritten rows: zero gradient
    stats = q.new_empty(lib.kfa_bwd_stats_bytes(n_seqs, q.shape[1], max_q) // 4, dtype=torch.float32)
    with torch.cuda.device(q.device):
        rc = lib.kfa_bwd_varlen(
            *(ctypes.byref(_lib.tensor4(_as4(t))) for t in (q, k, v, out, dout)),
            lse.data_ptr(),
            stats.data_ptr(),
            *(ctypes.byref(_lib.tensor4(_as4(t))) for t in (dq, dk, dv)),
            cu_seqlens_q.data_ptr(),
            cu_seqlens_k.data_ptr(),
            n_seqs,
            max_q,
            max_k,
            float(scale),
            int(block),
            _lib.dtype_code(q.dtype),
            _lib.status_word(q.device).data_ptr(),
            _lib.stream_ptr(q.device),
        )
    _lib.check(rc)
    return dq, dk, dv


@varlen_bwd_op.register_fake
def _(q, k, v, out, dout, lse, cu_seqlens_q, cu_seqlens_k, max_q, max_k, scale, block):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _varlen_setup(ctx, inputs, output):
    q, k, v, cu_q, cu_k, max_q, max_k, scale, block = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
    ctx.plan = (max_q, max_k)
    ctx.scale, ctx.block = scale, block
    ctx.mark_non_differentiable(lse)


def _varlen_backward(ctx, dout, dlse):
    q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
    dq, dk, dv = varlen_bwd_op(q, k, v, out, dout.contiguous(), lse, cu_q, cu_k, *ctx.plan, ctx.scale, ctx.block)
    return dq, dk, dv, None, None, None, None, None, None


varlen_fwd_op.register_autograd(_varlen_backward, setup_context=_varlen_setup)


def varlen_plan(
    cu_seqlens_q: Tensor, cu_seqlens_k: Tensor, heads: int = 0, kv_heads: int = 0, block: int = 0
) -> tuple[int, int, int]:
    """What a call needs to know about a batch of packed sequences on the HOST: (number of sequences,
    longest query length, longest key length). Reads ``cu_seqlens`` once (a device-to-host copy):
    build it outside CUDA-graph capture and reuse it for every call with the same lengths
    (reference: op.py:252-261; ``heads``, ``kv_heads``, ``block`` are accepted for signature
    compatibility, the plan does not depend on them). A sequence with queries but no keys is refused."""
    len_q = (cu_seqlens_q[1:] - cu_seqlens_q[:-1]).tolist()
    len_k = (cu_seqlens_k[1:] - cu_seqlens_k[:-1]).tolist()
    if len(len_q) != len(len_k) or not len_q:
        raise ValueError("varlen_plan: cu_seqlens_q and cu_seqlens_k must describe the same (non-zero) number of sequences")
    if min(len_q) < 0 or min(len_k) < 0:
        raise ValueError("varlen_plan: cu_seqlens must be non-decreasing")
    if any(nq > 0 and nk == 0 for nq, nk in zip(len_q, len_k)):
        raise ValueError("varlen_plan: a sequence with queries needs at least one key")
    return len(len_q), max(max(len_q), 1), max(max(len_k), 1)


def attention_varlen(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    cu_seqlens_q: Tensor,
    cu_seqlens_k: Tensor,
    scale: float | None = None,
    block_causal: int = 0,
    plan: tuple | None = None,
) -> Tensor:
    """Packed sequences, each its own attention problem: ``q [Tq, H, D]``, ``k / v [Tk, Hkv, D]``;
    sequence ``b`` is rows ``cu_seqlens[b] : cu_seqlens[b + 1]`` (int32 [B + 1] on the device).
    ``plan`` from ``varlen_plan`` (built here if None). Reference: op.py:264-289."""
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("attention_varlen: q, k, v must be [T, H, D]")
    _check(*(_as4(t) for t in (q, k, v)))
    if scale is None:
        scale = q.shape[-1] ** -0.5
    cu_seqlens_q, cu_seqlens_k = cu_seqlens_q.int(), cu_seqlens_k.int()
    if plan is None:
        plan = varlen_plan(cu_seqlens_q, cu_seqlens_k, q.shape[1], k.shape[1], block_causal)
    n_seqs, max_q, max_k = plan
    if cu_seqlens_q.numel() != n_seqs + 1 or cu_seqlens_k.numel() != n_seqs + 1:
        raise ValueError(f"attention_varlen: the plan is for {n_seqs} sequences")
    out, _ = varlen_fwd_op(q, k, v, cu_seqlens_q, cu_seqlens_k, int(max_q), int(max_k), float(scale), int(block_causal))
    return out
