"""GPU parity tests of boolean masks: ``attention(..., mask=)`` and ``pack_mask`` against the fp64
oracle, following the reference's mask tests (KohakuFA tests/test_attention.py:214-268, 347-360)."""

import pytest
import torch

from kohakufa_b200 import PackedMask, _lib, attention, pack_mask
from kohakufa_b200.mask import words_per_row
from oracle import reference as oracle

pytestmark = pytest.mark.gpu

TOL = 5e-3
BF16_TOL = 2e-2


def inputs(batch, heads, s_q, s_kv, dim=64, seed=0, dtype=torch.float16, kv_heads=None):
    gen = torch.Generator().manual_seed(seed)
    kv_heads = kv_heads or heads

    def projection(seq, h):
        return torch.randn(batch, seq, h, dim, generator=gen).to(dtype).cuda().transpose(1, 2).requires_grad_()

    dout = torch.randn(batch, heads, s_q, dim, generator=gen).to(dtype).cuda()
    return projection(s_q, heads), projection(s_kv, kv_heads), projection(s_kv, kv_heads), dout


def random_mask(shape, density, seed=3):
    gen = torch.Generator().manual_seed(seed)
    return (torch.rand(shape, generator=gen) < density).cuda()


def run(q, k, v, dout, **kwargs):
    for t in (q, k, v):
        t.grad = None
    out = attention(q, k, v, **kwargs)
    out.backward(dout)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return out, q.grad, k.grad, v.grad


def check(got, want, tol=TOL):
    for name, g, w in zip(("out", "dq", "dk", "dv"), got, want):
        assert bool(torch.isfinite(g).all()), name
        m = oracle.metrics(g, w)
        assert m["rel_err"] < tol, f"{name}: {m}"


def test_pack_mask_words():
    """Bit c % 32 of word c // 32 of a row is key c; the transposed words the same over queries;
    rows padded with zero bits to whole 128-wide tiles."""
    mask = random_mask((2, 3, 269, 517), 0.5)
    packed = pack_mask(mask, 2, 3, 269, 517)
    assert packed.words.shape == (2, 3, 269, words_per_row(517)) and packed.words_t.shape == (2, 3, 517, words_per_row(269))

    def unpack(words, n):
        bits = (words.unsqueeze(-1) >> torch.arange(32, device=words.device)) & 1
        flat = bits.flatten(-2)
        assert int(flat[..., n:].sum()) == 0  # padding
        return flat[..., :n].bool()

    assert torch.equal(unpack(packed.words, 517), mask)
    assert torch.equal(unpack(packed.words_t, 269), mask.transpose(-1, -2))
    assert packed.tiles.shape == (2, 3, 3, 5) and bool((packed.tiles != 0).all())  # dense random mask: no empty tile


def structured_mask(kind, s_q, s_kv):
    r = torch.arange(s_q, device="cuda")[:, None]
    c = torch.arange(s_kv, device="cuda")[None, :]
    if kind == "window":  # sliding window of 200 keys behind the diagonal
        return (c <= r) & (c > r - 200)
    if kind == "block_diagonal":  # documents of 300 tokens
        return (r // 300) == (c // 300)
    if kind == "prefix":  # everybody sees the first 100 keys, plus its own 128-block
        return (c < 100) | ((r // 128) == (c // 128))
    if kind == "last_rows_blind":  # the last 300 query rows see nothing
        return (r < s_q - 300) & (c <= r)
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["window", "block_diagonal", "prefix", "last_rows_blind"])
@pytest.mark.parametrize("dim,heads,kv_heads", [(64, 2, 2), (128, 4, 2)])
def test_mask_with_empty_tiles(kind, dim, heads, kv_heads):
    """Masks with whole 128 x 128 tiles hidden: the kernels skip them (table of non-empty tiles) and give
    the same result as the oracle, which sees the dense mask."""
    s_q, s_kv = 1100, 1300
    mask = structured_mask(kind, s_q, s_kv)
    packed = pack_mask(mask, 1, heads, s_q, s_kv)
    dense_any = torch.nn.functional.pad(mask, (0, -s_kv % 128, 0, -s_q % 128)).reshape(9, 128, 11, 128).any(3).any(1)
    assert torch.equal(packed.tiles[0, 0] != 0, dense_any) and not bool(dense_any.all())
    q, k, v, dout = inputs(1, heads, s_q, s_kv, dim=dim, kv_heads=kv_heads)
    got = run(q, k, v, dout, mask=packed)
    check(got, oracle.attention_fp64(q, k, v, dout, dim**-0.5, mask=mask, groups=heads // kv_heads))
    if kind == "last_rows_blind":
        assert float(got[0].detach()[:, :, -300:].abs().max()) == 0.0 and float(got[1][:, :, -300:].abs().max()) == 0.0


def test_skipping_tiles_does_not_change_the_bits():
    """The same mask with and without the tile table: identical results (hidden tiles contribute exact
    zeros when they are visited)."""
    mask = structured_mask("window", 1100, 1300)
    q, k, v, dout = inputs(2, 2, 1100, 1300)
    packed = pack_mask(mask, 2, 2, 1100, 1300)
    a = run(q, k, v, dout, mask=packed)
    packed.tiles.fill_(1)  # visit everything
    b = run(q, k, v, dout, mask=packed)
    for name, x, y in zip(("out", "dq", "dk", "dv"), a, b):
        assert torch.equal(x, y), name


@pytest.mark.parametrize(
    "shape,mask_shape,density",
    [
        ((2, 3, 269, 269), "full", 0.5),
        ((2, 3, 269, 269), "broadcast", 0.3),
        ((2, 2, 131, 517), "full", 0.7),
        ((1, 2, 1000, 1000), "head", 0.05),
    ],
    ids=str,
)
def test_mask(shape, mask_shape, density):
    batch, heads, s_q, s_kv = shape
    m_shape = {"full": (batch, heads, s_q, s_kv), "broadcast": (1, 1, s_q, s_kv), "head": (1, heads, s_q, s_kv)}[mask_shape]
    mask = random_mask(m_shape, density)
    q, k, v, dout = inputs(*shape)
    check(run(q, k, v, dout, mask=mask), oracle.attention_fp64(q, k, v, dout, 64**-0.5, mask=mask))


@pytest.mark.parametrize("dim,dtype,tol", [(128, torch.bfloat16, BF16_TOL), (128, torch.float16, TOL), (64, torch.bfloat16, BF16_TOL),
                                           (32, torch.float16, TOL), (112, torch.bfloat16, BF16_TOL)])
def test_mask_dims_and_dtypes(dim, dtype, tol):
    q, k, v, dout = inputs(1, 2, 300, 389, dim=dim, dtype=dtype)
    mask = random_mask((1, 2, 300, 389), 0.5)
    check(run(q, k, v, dout, mask=mask), oracle.attention_fp64(q, k, v, dout, dim**-0.5, mask=mask), tol=tol)


def test_mask_key_padding_and_empty_rows():
    """[B, 1, 1, Skv] key padding, plus rows that see no key at all (output 0, finite gradients)."""
    q, k, v, dout = inputs(2, 4, 300, 300)
    lengths = torch.tensor([300, 157], device="cuda")
    mask = (torch.arange(300, device="cuda")[None, :] < lengths[:, None])[:, None, None, :]
    mask = mask.expand(2, 4, 300, 300).clone()
    mask[:, :, 10:20] = False  # empty rows
    got = run(q, k, v, dout, mask=mask)
    assert all(bool(torch.isfinite(g).all()) for g in got)
    assert bool((got[0][:, :, 10:20] == 0).all()) and bool((got[1][:, :, 10:20] == 0).all())
    check(got, oracle.attention_fp64(q, k, v, dout, 64**-0.5, mask=mask))


def test_mask_broadcast_key_padding_without_copy():
    """A [B, 1, 1, Skv] mask expanded (stride 0) over heads and rows is packed as it is."""
    q, k, v, dout = inputs(2, 2, 200, 333)
    lengths = torch.tensor([333, 90], device="cuda")
    mask = (torch.arange(333, device="cuda")[None, :] < lengths[:, None])[:, None, None, :].expand(2, 1, 200, 333)
    check(run(q, k, v, dout, mask=mask), oracle.attention_fp64(q, k, v, dout, 64**-0.5, mask=mask))


def test_mask_equals_causal():
    """A lower-triangular mask and causal=True select the same visible pairs (reference test:
    tests/test_attention.py:261-268)."""
    q, k, v, dout = inputs(1, 2, 600, 600)
    causal = torch.ones(600, 600, dtype=torch.bool, device="cuda").tril()
    masked = run(q, k, v, dout, mask=causal)
    native = run(q, k, v, dout, causal=True)
    for name, a, b in zip(("out", "dq", "dk", "dv"), masked, native):
        assert oracle.metrics(a, b)["rel_err"] < 1e-3, name


def test_mask_gqa_bf16():
    q, k, v, dout = inputs(2, 8, 269, 269, dtype=torch.bfloat16, kv_heads=2)
    mask = random_mask((2, 8, 269, 269), 0.5)
    got = run(q, k, v, dout, mask=mask)
    check(got, oracle.attention_fp64(q, k, v, dout, 64**-0.5, groups=4, mask=mask), tol=BF16_TOL)


def test_packed_mask_reuse():
    """pack_mask once, reuse across calls: identical to passing the bool mask (every gradient, dQ
    included: nothing here is reduced in arbitrary order)."""
    q, k, v, dout = inputs(2, 3, 600, 600)
    mask = random_mask((2, 1, 600, 600), 0.4)
    packed = pack_mask(mask, 2, 3, 600, 600)
    assert isinstance(packed, PackedMask)
    a = run(q, k, v, dout, mask=packed)
    b = run(q, k, v, dout, mask=mask)
    for name, x, y in zip(("out", "dq", "dk", "dv"), a, b):
        assert torch.equal(x, y), name


def test_mask_argument_errors():
    q, k, v, _ = inputs(1, 2, 64, 64)
    with pytest.raises(ValueError):
        attention(q, k, v, causal=True, mask=torch.ones(64, 64, dtype=torch.bool, device="cuda"))
    with pytest.raises(TypeError):
        attention(q, k, v, mask=torch.ones(64, 64, device="cuda"))
    with pytest.raises(ValueError):
        attention(q, k, v, mask=torch.ones(64, 65, dtype=torch.bool, device="cuda"))
    with pytest.raises(ValueError):  # packed for another shape
        attention(q, k, v, mask=pack_mask(torch.ones(32, 64, dtype=torch.bool, device="cuda"), 1, 2, 32, 64))


def test_mask_compiled_and_all_visible_equals_dense():
    """An all-True mask gives the dense result bit for bit; the masked ops trace under torch.compile."""
    q, k, v, dout = inputs(1, 2, 300, 300)
    from kohakufa_b200 import set_backward

    packed = pack_mask(torch.ones(300, 300, dtype=torch.bool, device="cuda"), 1, 2, 300, 300)
    set_backward("split")  # masks run the split backward kernels: compare like with like
    try:
        dense = run(q, k, v, dout)
    finally:
        set_backward("auto")
    masked = run(q, k, v, dout, mask=packed)
    for a, b in zip(dense, masked):
        assert torch.equal(a, b)
    fn = torch.compile(lambda q, k, v: attention(q, k, v, mask=packed), fullgraph=True)
    assert torch.equal(fn(q, k, v), masked[0])
    # a bool mask given directly: the packing is a custom op too, so this traces as well
    ones = torch.ones(300, 300, dtype=torch.bool, device="cuda")
    fn2 = torch.compile(lambda q, k, v, m: attention(q, k, v, mask=m), fullgraph=True)
    assert torch.equal(fn2(q, k, v, ones), masked[0])
