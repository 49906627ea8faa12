"""Boolean attention masks packed for the kernels: 32 keys per int32 word along each query row (read by
the forward and the dQ kernel) and 32 queries per word along each key row (read by the dK / dV kernel),
padded with zero bits to whole 128-wide tiles.

Same interface and word format as the reference's ``PackedMask`` / ``pack_mask`` (KohakuFA
``src/kohakufa/mask.py:13-128``); the packing is one CUDA kernel of ``libkfa.so`` (``kfa_pack_mask``)
instead of a Triton kernel. In place of the reference's tile classes and host-built tile lists
(mask.py:74-122) the packing fills a table with one int per (128 queries x 128 keys) tile, nonzero where
the tile holds a visible pair; the kernels list the tiles they visit from it and skip the rest.
"""

import ctypes

import torch
from torch import Tensor

from kohakufa_b200 import _lib

TILE = 128


def normalize(mask: Tensor, batch: int, heads: int, s_q: int, s_kv: int) -> Tensor:
    """A bool mask broadcastable to ``[B, H, Sq, Skv]`` (True = visible) as 4D with batch / head
    dimensions of size 1 or B / H (reference mask.py:13-29: same exceptions)."""
    if mask.dtype != torch.bool:
        raise TypeError("mask: a boolean tensor (True = the key is visible)")
    while mask.dim() < 4:
        mask = mask.unsqueeze(0)
    if mask.shape[-2:] != (s_q, s_kv) or mask.shape[0] not in (1, batch) or mask.shape[1] not in (1, heads):
        raise ValueError(f"mask {tuple(mask.shape)} does not broadcast to {(batch, heads, s_q, s_kv)}")
    return mask


def words_per_row(n: int) -> int:
    """int32 words of a row of ``n`` bits, padded to whole 128-bit tiles."""
    return 4 * (-(-n // TILE))


@torch.library.custom_op("kohakufa_b200::pack_mask", mutates_args=(), device_types="cuda")
def pack_mask_op(mask: Tensor, s_q: int, s_kv: int) -> tuple[Tensor, Tensor, Tensor]:
    """words, words_t, tiles of a ``[Bm, Hm, Sq, Skv]`` bool mask (True = visible), any strides."""
    mask_bytes = mask.view(torch.uint8)
    bm, hm = mask_bytes.shape[:2]
    dev = mask_bytes.device
    words = torch.empty(bm, hm, s_q, words_per_row(s_kv), dtype=torch.int32, device=dev)
    words_t = torch.empty(bm, hm, s_kv, words_per_row(s_q), dtype=torch.int32, device=dev)
    tiles = torch.zeros(bm, hm, -(-s_q // TILE), -(-s_kv // TILE), dtype=torch.int32, device=dev)
    lib = _lib.load()
    strides = (ctypes.c_int64 * 4)(*mask_bytes.stride())
    with torch.cuda.device(dev):
        rc = lib.kfa_pack_mask(
            mask_bytes.data_ptr(), strides, bm, hm, s_q, s_kv, words.data_ptr(), words_t.data_ptr(),
            tiles.data_ptr(), _lib.stream_ptr(dev),
        )  # fmt: skip
    _lib.check(rc)
    return words, words_t, tiles


@pack_mask_op.register_fake
def _(mask, s_q, s_kv):
    bm, hm = mask.shape[:2]
    new = lambda *shape: mask.new_empty(*shape, dtype=torch.int32)  # noqa: E731
    return (new(bm, hm, s_q, words_per_row(s_kv)), new(bm, hm, s_kv, words_per_row(s_q)),
            new(bm, hm, -(-s_q // TILE), -(-s_kv // TILE)))  # fmt: skip


class PackedMask:
    """A boolean mask packed once for the kernels (words, transposed words, table of non-empty tiles),
    reusable across calls with the same mask and shape (e.g. every layer of a model)."""

    def __init__(self, mask: Tensor, batch: int, heads: int, s_q: int, s_kv: int) -> None:
        dense = normalize(mask, batch, heads, s_q, s_kv)
        if not dense.is_cuda:
            raise ValueError("mask: a CUDA tensor (there is no CPU path)")
        self.shape = (batch, heads, s_q, s_kv)
        self.words, self.words_t, self.tiles = pack_mask_op(dense, s_q, s_kv)


def pack_mask(mask: Tensor, batch: int, heads: int, s_q: int, s_kv: int) -> PackedMask:
    """Pack ``mask`` (bool, broadcastable to ``[B, H, Sq, Skv]``, True = visible) once; pass the result
    as ``attention(..., mask=packed)``."""
    return PackedMask(mask, batch, heads, s_q, s_kv)


def mask_words(words: Tensor, batch: int, heads: int) -> "_lib.KfaMaskWords":
    """The library's descriptor of ``words [Bm, Hm, rows, row_words]`` (size-1 dimensions broadcast)."""
    assert words.dtype == torch.int32 and words.dim() == 4 and words.stride(3) == 1
    d = _lib.KfaMaskWords()
    d.words = words.data_ptr()
    d.stride_batch = words.stride(0) if words.shape[0] > 1 else 0
    d.stride_head = words.stride(1) if words.shape[1] > 1 else 0
    d.stride_row = words.stride(2)
    return d


def mask_tiles(tiles: Tensor) -> "_lib.KfaMaskTiles":
    """The library's descriptor of the tile table ``[Bm, Hm, ceil(Sq / 128), ceil(Skv / 128)]``."""
    assert tiles.dtype == torch.int32 and tiles.dim() == 4 and tiles.is_contiguous()
    d = _lib.KfaMaskTiles()
    d.any = tiles.data_ptr()
    d.stride_batch = tiles.stride(0) if tiles.shape[0] > 1 else 0
    d.stride_head = tiles.stride(1) if tiles.shape[1] > 1 else 0
    return d
