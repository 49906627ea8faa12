"""Seeded synthetic inputs of the five benchmark configurations, and the FLOP convention.

Inputs are generated on the CPU (``torch.Generator().manual_seed``) in fp32, rounded to the 16-bit
dtype, then moved to the device: the CPU oracle and the kernels see identical bits on any machine.
Q, K, V are ``[B, S, H, D]`` storage viewed as ``[B, H, S, D]`` (how a projection layer produces them,
and how the reference's tests build theirs, KohakuFA tests/test_attention.py:15-30).

    C1  dense        fp16  B2  H4  S512   D64
    C2  dense, large logits (~1e5), near-one-hot rows, fp16 / bf16  B32 H12 S201 D64
    C3  causal       bf16  B4  H32 S8192  D128
    C4  block-causal P=256 fp16 B8 H16 S4096 D64   (+ dense S=4100)
    C5  causal       bf16  B1  H32 S131072 D128    (context-parallel ring across GPUs)
"""

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Config:
    name: str
    batch: int
    heads: int
    seq: int
    dim: int
    dtype: torch.dtype
    block: int  # 0 dense, 1 causal, P block-causal
    seed: int
    std: float = 1.0
    large_logits: bool = False

    @property
    def scale(self) -> float:
        return self.dim**-0.5


CONFIGS = {
    "C1": Config("C1", 2, 4, 512, 64, torch.float16, 0, 0),
    "C2": Config("C2", 32, 12, 201, 64, torch.float16, 0, 1, large_logits=True),
    "C2-bf16": Config("C2-bf16", 32, 12, 201, 64, torch.bfloat16, 0, 1, large_logits=True),
    "C3": Config("C3", 4, 32, 8192, 128, torch.bfloat16, 1, 2, std=0.5),
    "C4": Config("C4", 8, 16, 4096, 64, torch.float16, 256, 3),
    "C4-dense4100": Config("C4-dense4100", 8, 16, 4100, 64, torch.float16, 0, 3),
    "C5": Config("C5", 1, 32, 131072, 128, torch.bfloat16, 1, 4, std=0.5),
}


def visible_pairs(s_q: int, s_kv: int, block: int) -> int:
    """Number of (query, key) pairs with ``key // block <= query // block`` (all pairs if dense)."""
    if block == 0:
        return s_q * s_kv
    total = 0
    full, rem = divmod(s_q, block)
    for frame in range(full):
        total += block * min((frame + 1) * block, s_kv)
    total += rem * min((full + 1) * block, s_kv)
    return total


def attention_flops(batch, heads, s_q, s_kv, dim, block=0, backward=True) -> float:
    """Algorithmic FLOPs in the reference's convention (KohakuFA benchmarks/speed.py:21-26, 93, 108):
    forward 4 B H D x visible pairs; forward + backward 3.5 x that (2 + 5 matmuls). Recomputation
    inside the kernels is never counted."""
    fwd = 4.0 * batch * heads * dim * visible_pairs(s_q, s_kv, block)
    return fwd * (3.5 if backward else 1.0)


def _bshd(x: torch.Tensor) -> torch.Tensor:
    return x.transpose(1, 2)


PIECE_ROWS = 8192  # granularity of make_piecewise_inputs: one seed per 8192 rows of the sequence


def make_piecewise_inputs(cfg: Config, row_ranges, device="cpu", device_rng=False):
    """q, k, v, dout for the given row ranges of ``cfg``'s sequence, generated piece by piece (one seed
    per PIECE_ROWS rows), so that a rank of a context-parallel run builds only its own rows and every
    world size sees the same global tensors. ``row_ranges``: list of (start, stop), multiples of
    PIECE_ROWS. Returns ``[B, H, rows, D]`` views of ``[B, rows, H, D]`` storage.
    ``device_rng``: draw the numbers with ``device``'s own generator (fast for long sequences; the values
    then depend on the GPU model, which is fine where the check is computed from the same tensors)."""
    outs = []
    rng_device = device if device_rng else "cpu"
    for which in range(4):
        parts = []
        for start, stop in row_ranges:
            assert start % PIECE_ROWS == 0 and stop % PIECE_ROWS == 0
            for piece in range(start // PIECE_ROWS, stop // PIECE_ROWS):
                gen = torch.Generator(device=rng_device).manual_seed(1_000_003 * (cfg.seed + 1) + 4 * piece + which)
                x = torch.randn(cfg.batch, PIECE_ROWS, cfg.heads, cfg.dim, generator=gen, device=rng_device) * cfg.std
                parts.append(x.to(cfg.dtype))
        outs.append(torch.cat(parts, dim=1).to(device).transpose(1, 2))
    return tuple(outs)


def make_inputs(cfg: Config, batch=None, heads=None, seq=None, device="cpu", seed_offset=0):
    """q, k, v, dout for ``cfg`` (optionally a smaller batch / head count / length of the same
    recipe). Views of [B, S, H, D] storage, already rounded to ``cfg.dtype``."""
    b = cfg.batch if batch is None else batch
    h = cfg.heads if heads is None else heads
    s = cfg.seq if seq is None else seq
    gen = torch.Generator().manual_seed(cfg.seed + 1000 * seed_offset)
    if cfg.large_logits:
        q, k, v, dout = _large_logit_inputs(b, h, s, cfg.dim, cfg.dtype, gen)
    else:
        q, k, v, dout = (
            (torch.randn(b, s, h, cfg.dim, generator=gen) * cfg.std).to(cfg.dtype) for _ in range(4)
        )
    return tuple(_bshd(t).to(device) for t in (q, k, v, dout))


def _large_logit_inputs(b, s_heads, s, dim, dtype, gen):
    """Near-one-hot rows with max logit ~1e5 and a runner-up within ~1e1 (ViT-shaped, standing in
    for the pretrained layer the reference's precision study probes, KohakuFA README.md:18-25).

    Query rows come in pairs: row 2i+1 is row 2i with a few coordinates moved up by one unit in the
    last place. Each row gets a planted key alpha * q_row with alpha = 1e5 sqrt(D) / |q_2i|^2, so a
    row's own key and its twin's key score ~1e5 and differ by only a few units."""
    h = s_heads
    q = torch.randn(b, s, h, dim, generator=gen).clamp_(-4.0, 4.0).to(dtype)
    nudges = 4 if dtype == torch.float16 else 1
    pairs = s // 2
    even = q[:, 0 : 2 * pairs : 2].clone()
    odd = even.clone()
    idx = torch.rand(b, pairs, h, dim, generator=gen).argsort(-1)[..., :nudges]
    # one unit in the last place of the 16-bit format, towards +inf: step the bit pattern
    bits = even.view(torch.int16)
    ulp_up = torch.where(even >= 0, bits + 1, bits - 1).view(dtype)
    ulp_up = torch.where(even == 0, torch.zeros_like(even), ulp_up)  # keep zeros (a subnormal nudge is lost)
    odd.scatter_(-1, idx, ulp_up.gather(-1, idx))
    q[:, 0 : 2 * pairs : 2] = even
    q[:, 1 : 2 * pairs : 2] = odd
    qf = q.float()
    norm2 = (qf[:, 0 : 2 * pairs : 2] ** 2).sum(-1, keepdim=True)
    alpha = 1e5 * dim**0.5 / norm2
    k = torch.randn(b, s, h, dim, generator=gen)
    k[:, 0 : 2 * pairs : 2] = alpha * qf[:, 0 : 2 * pairs : 2]
    k[:, 1 : 2 * pairs : 2] = alpha * qf[:, 1 : 2 * pairs : 2]
    k = k.to(dtype)
    v = torch.randn(b, s, h, dim, generator=gen).to(dtype)
    dout = torch.randn(b, s, h, dim, generator=gen).to(dtype)
    return q, k, v, dout


def balanced_large_logit_inputs(b, h, s, dim, dtype, logit=1e5, clusters=16, jitter=1e-3, seed=0):
    """The reference's own large-logit generator (KohakuFA benchmarks/precision.py:27-44): queries and
    keys are jittered copies of a few unit-norm cluster centres, both scaled by
    sqrt(logit * sqrt(D)), so the magnitude is split evenly between q and k."""
    gen = torch.Generator().manual_seed(seed)
    centers = torch.randn(b, h, clusters, dim, generator=gen)
    centers = centers / centers.norm(dim=-1, keepdim=True)
    pick = torch.randint(0, clusters, (b, h, s), generator=gen)
    base = torch.gather(centers, 2, pick[..., None].expand(-1, -1, -1, dim))
    radius = (logit * dim**0.5) ** 0.5

    def around(t):
        return (radius * (t + jitter * torch.randn(t.shape, generator=gen))).to(dtype)

    q, k = around(base), around(base)
    v = torch.randn(base.shape, generator=gen).to(dtype)
    dout = torch.randn(base.shape, generator=gen).to(dtype)
    return q, k, v, dout
