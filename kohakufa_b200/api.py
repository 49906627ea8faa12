"""``attention`` and ``attention_varlen``: the calls a user of the package makes.

They take the arguments, defaults and error conditions of the reference's entry points
(KohakuFA ``src/kohakufa/api.py:56-146``), turn them into what the kernels understand (a frame size,
a 16-bit compute dtype, a head dim the kernels are built for) and hand over to the custom ops in
``kohakufa_b200.op``, which launch ``libkfa.so``. Nothing is computed here except the optional
key centring, which is a handful of fp32 torch reductions.
"""

import torch
from torch import Tensor

from kohakufa_b200 import op as _op
from kohakufa_b200.op import varlen_plan  # noqa: F401  (part of the public surface)

COMPUTE_DTYPES = (torch.float16, torch.bfloat16)
MAX_HEAD_DIM = _op.MAX_KERNEL_DIM


def _frame_size(causal: bool, block_causal: int) -> int:
    """The one integer the kernels mask by: 0 dense, 1 token-causal, P frames of P tokens."""
    if causal and block_causal not in (0, 1):
        raise ValueError("causal is block_causal=1: give one of them")
    return 1 if causal else int(block_causal)


def _fit_head_dim(*tensors: Tensor) -> tuple[Tensor, ...]:
    """Zero-extends the last dimension to the next head dim a kernel exists for.

    Added zero columns contribute nothing to ``q . k``, and the output columns they produce are
    sliced away by the caller, which also keeps the softmax scale of the true head dim, so the
    result is exact (the reference widens the same way, api.py:18-29)."""
    dim = tensors[0].shape[-1]
    if not 1 <= dim <= MAX_HEAD_DIM:
        raise ValueError(f"head_dim {dim}: 1 .. {MAX_HEAD_DIM} supported")
    target = _op.kernel_dim_for(dim)
    if target == dim:
        return tensors
    return tuple(torch.nn.functional.pad(t, (0, target - dim)) for t in tensors)


def _remove_key_mean(k: Tensor, dtype: torch.dtype, cu_seqlens: Tensor | None = None) -> Tensor:
    """``k`` minus the average key of its sequence, computed in fp32 and rounded once to ``dtype``.

    Every score of a query row then moves by one common amount, which softmax ignores, so outputs
    are unchanged while the large component all keys share never reaches the 16-bit rounding;
    autograd routes ``-mean(dK)`` back (reference api.py:32-53).

    Dense input ``[B, Hkv, Skv, D]``: one average per (batch, head), over dim -2. Packed input
    ``[Tk, Hkv, D]`` with ``cu_seqlens``: one average per (sequence, head); sequence membership of a
    row is derived on the device, so no length is read back to the host."""
    k32 = k.float()
    if cu_seqlens is None:
        return (k32 - k32.mean(dim=-2, keepdim=True)).to(dtype)
    lengths = cu_seqlens[1:] - cu_seqlens[:-1]
    owner = torch.repeat_interleave(
        torch.arange(lengths.numel(), device=k.device), lengths.long(), output_size=k.shape[0]
    )
    totals = k32.new_zeros(lengths.numel(), *k.shape[1:]).index_add_(0, owner, k32)
    mean = totals / lengths.clamp(min=1).to(torch.float32).view(-1, 1, 1)
    return (k32 - mean[owner]).to(dtype)


def attention(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    *,
    causal: bool = False,
    block_causal: int = 0,
    scale: float | None = None,
    mask=None,
    compute_dtype: torch.dtype | None = None,
    center_keys: bool = False,
) -> Tensor:
    """Scaled dot-product attention, forward and (through autograd) backward, on the B200 kernels.

    ``q`` is ``[B, H, Sq, D]``; ``k`` and ``v`` are ``[B, Hkv, Skv, D]`` where ``Hkv`` divides ``H``
    (each K / V head serves ``H // Hkv`` consecutive query heads). Transposed views of
    ``[B, S, H, D]`` projections are taken as they are: only the last dim must be contiguous and
    the other strides 16-byte multiples.

    Visibility, one of:
      * nothing: every query sees every key;
      * ``causal=True``: query ``r`` sees keys ``0 .. r`` (rows and columns both count from 0 when
        ``Sq != Skv``);
      * ``block_causal=P``: tokens come in frames of ``P``; a query sees the keys of its own and of
        earlier frames (``c // P <= r // P``). ``causal`` is the case ``P = 1``;
      * ``mask``: a bool tensor that broadcasts to ``[B, H, Sq, Skv]`` (True = visible), or the result
        of ``pack_mask`` to pay for the packing once. Cannot be combined with the two above. A query
        with no visible key gets a zero output row and zero gradients.

    ``scale`` defaults to ``D ** -0.5`` of the head dim passed in. ``compute_dtype`` is the 16-bit
    dtype the tensor cores see; inputs of another dtype are cast to it (fp16 unless they already are
    fp16 / bf16) and the result is cast back. ``center_keys`` subtracts each (batch, head)'s mean key
    in fp32 before that cast (see ``_remove_key_mean``): same function, better conditioned.

    Returns ``[B, H, Sq, D]`` in the dtype of ``q``, laid out as ``[B, Sq, H, D]`` in memory.
    """
    frame = _frame_size(causal, block_causal)
    if compute_dtype is None:
        compute_dtype = q.dtype if q.dtype in COMPUTE_DTYPES else torch.float16
    if compute_dtype not in COMPUTE_DTYPES:
        raise TypeError(f"compute_dtype {compute_dtype}: one of {COMPUTE_DTYPES}")
    result_dtype, head_dim = q.dtype, q.shape[-1]
    if center_keys:
        k = _remove_key_mean(k, compute_dtype)
    q, k, v = _fit_head_dim(*(t.to(compute_dtype) for t in (q, k, v)))
    if mask is not None and frame:
        raise ValueError("give a mask or causal / block_causal, not both (fold them in)")
    softmax_scale = head_dim**-0.5 if scale is None else scale
    out = _op.attention(q, k, v, softmax_scale, frame, mask)[..., :head_dim]
    return out.to(result_dtype) if out.dtype != result_dtype else out


def attention_varlen(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    cu_seqlens_q: Tensor,
    cu_seqlens_k: Tensor,
    *,
    causal: bool = False,
    block_causal: int = 0,
    scale: float | None = None,
    plan: tuple | None = None,
    center_keys: bool = False,
) -> Tensor:
    """Attention over a packed batch: sequences of different lengths stored back to back, each
    attended to on its own, with no padding rows computed (reference api.py:114-146).

    ``q`` is ``[Tq, H, D]``, ``k`` / ``v`` are ``[Tk, Hkv, D]`` (fp16 or bf16); int32 ``cu_seqlens_*``
    of length ``B + 1`` give the row range ``[cu[b], cu[b + 1])`` of sequence ``b``. ``causal`` and
    ``block_causal`` are applied inside every sequence. ``plan`` is what ``varlen_plan`` returned for
    these lengths; passing it keeps this call free of device-to-host reads (needed under CUDA-graph
    capture), otherwise it is built here. ``center_keys`` removes each sequence's own mean key.
    """
    frame = _frame_size(causal, block_causal)
    head_dim = q.shape[-1]
    if center_keys:
        k = _remove_key_mean(k, k.dtype, cu_seqlens_k)
    q, k, v = _fit_head_dim(q, k, v)
    out = _op.attention_varlen(
        q,
        k,
        v,
        cu_seqlens_q,
        cu_seqlens_k,
        scale=head_dim**-0.5 if scale is None else scale,
        block_causal=frame,
        plan=plan,
    )
    return out[..., :head_dim]
