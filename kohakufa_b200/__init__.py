"""kohakufa_b200: flash attention forward + backward for NVIDIA B200 (sm_100a), a drop-in for the
``kohakufa.attention`` entry point of KohakuFA with hand-written CUDA behind a C ABI.

    from kohakufa_b200 import attention
    out = attention(q, k, v, causal=True)  # q [B, H, Sq, D], k / v [B, H, Skv, D]

    out = attention_varlen(q, k, v, cu_seqlens, cu_seqlens, causal=True)  # packed [T, H, D]
    out = attention(q, k, v, mask=pack_mask(mask, B, H, Sq, Skv))  # boolean mask, packed once

Same exports as the reference (``src/kohakufa/__init__.py:12``), plus a few of this package's own:
``set_backward`` / ``set_deterministic`` (which backward kernels run; bit-reproducible gradients), ``check_status`` / ``reset_status`` (the device-side
health word, see ``check_status``).
"""

from kohakufa_b200._lib import check_status, reset_status
from kohakufa_b200.api import attention, attention_varlen, varlen_plan
from kohakufa_b200.mask import PackedMask, pack_mask
from kohakufa_b200.op import get_backward, is_deterministic, set_backward, set_deterministic

__all__ = [
    "PackedMask",
    "attention",
    "attention_varlen",
    "check_status",
    "get_backward",
    "is_deterministic",
    "pack_mask",
    "reset_status",
    "set_backward",
    "set_deterministic",
    "varlen_plan",
]
__version__ = "0.1.0"
