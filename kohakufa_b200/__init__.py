"""kohakufa_b200: flash attention forward + backward for NVIDIA B200 (sm_100a), a drop-in for the
``kohakufa.attention`` entry point of KohakuFA with hand-written CUDA behind a C ABI.

    from kohakufa_b200 import attention
    out = attention(q, k, v, causal=True)  # q [B, H, Sq, D], k / v [B, H, Skv, D]

    out = attention_varlen(q, k, v, cu_seqlens, cu_seqlens, causal=True)  # packed [T, H, D]

``pack_mask`` and ``PackedMask`` (the reference's other exports, ``src/kohakufa/__init__.py:12``)
are not built: they raise ``NotImplementedError``.
"""

from kohakufa_b200.api import attention, attention_varlen, varlen_plan


def _not_built(name):
    def stub(*args, **kwargs):
        raise NotImplementedError(f"kohakufa_b200.{name} is not built (only attention() is)")

    stub.__name__ = name
    return stub


pack_mask = _not_built("pack_mask")


class PackedMask:
    def __init__(self, *args, **kwargs):
        raise NotImplementedError("kohakufa_b200.PackedMask is not built (only attention() is)")


__all__ = ["PackedMask", "attention", "attention_varlen", "pack_mask", "varlen_plan"]
__version__ = "0.1.0"
