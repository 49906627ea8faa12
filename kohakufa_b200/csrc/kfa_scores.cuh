// kfa_scores: the raw scores S = Q K^T (no scale, no mask) written out as fp32, produced by the same
// tensor-core instruction sequence as in the attention kernels: both operands K-major in 128-byte
// swizzled shared memory, one tcgen05.mma (kind::f16, fp32 accumulate) per 16 elements of the head
// dim, in ascending order. A diagnostic: it shows what the kernels' softmax actually sees, which is
// not the correctly rounded dot product (the tensor core adds the products of a step with a
// truncating fp32 adder), so that an accuracy floor can be computed from the hardware's own scores.
// The reference has no counterpart; its emulation assumes correctly rounded scores
// (benchmarks/dinov3_backward.py:236). Included at the end of kfa_api.cu (uses its helpers).
#pragma once

namespace kfa {

struct ScoreParams {
  float* out;  // [B, H, Sq, Skv] contiguous
  int H, Sq, Skv, group;
  int n_q128, n_k128;
  int* status;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(128, 1)
kfa_scores_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const ScoreParams p) {
  constexpr int CH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base, sK = smem_base + CH * TILE_BYTES_64;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * CH * TILE_BYTES_64);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const uint32_t bar0 = smem_u32(bars);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int kt = blockIdx.x % p.n_k128;
  const int qt = (blockIdx.x / p.n_k128) % p.n_q128;
  const int bh = blockIdx.x / (p.n_k128 * p.n_q128);
  const int b = bh / p.H, h = bh % p.H;
  if (tid == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    *s_abort = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(s_tmem), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const Ctl ctl{s_abort, p.status};
  bool ok = (*s_abort == 0);
  if (ok && tid == 0) {
    mbar_expect_tx(bar0, 2 * CH * TILE_BYTES_64);
    for (int ch = 0; ch < CH; ++ch) {
      tma_load_4d(sQ + ch * TILE_BYTES_64, &tmQ, bar0, ch * 64, qt * 128, h, b);
      tma_load_4d(sK + ch * TILE_BYTES_64, &tmK, bar0, ch * 64, kt * 128, h / p.group, b);
    }
    if (mbar_wait(bar0, 0, ctl, 94)) {
      tc_fence_after();
      constexpr uint32_t IDESC = make_idesc(BF16, false, 128, 128);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk >> 2) * TILE_BYTES_64 + (kk & 3) * 32;
        umma_ss(tmem, make_sdesc(sQ + off, 16, 1024), make_sdesc(sK + off, 16, 1024), IDESC, kk > 0);
      }
      umma_commit(bar0 + 8);
    } else {
      mbar_drain(bar0, 0);  // gave up: the copies still have to land before the CTA leaves
    }
  }
  if (ok) ok = mbar_wait_warp(bar0 + 8, 0, ctl, 95);
  if (ok) {
    tc_fence_after();
    const int row = qt * 128 + tid;
    const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    float* orow = p.out + (static_cast<long long>(bh) * p.Sq + row) * p.Skv + kt * 128;
    for (int c0 = 0; c0 < 128; c0 += 32) {
      float s[32];
      tmem_ld32(taddr + c0, reinterpret_cast<uint32_t*>(s));
      tmem_wait_ld();
      if (row < p.Sq)
        for (int i = 0; i < 32; ++i)
          if (kt * 128 + c0 + i < p.Skv) orow[c0 + i] = s[i];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 128);
  }
}

}  // namespace kfa

namespace {

template <int D, bool BF16>
int launch_scores(const CUtensorMap& mq, const CUtensorMap& mk, const kfa::ScoreParams& p, long long grid, cudaStream_t s) {
  auto kern = kfa::kfa_scores_kernel<D, BF16>;
  constexpr int smem = 2 * (D / 64) * kfa::TILE_BYTES_64 + 1024 + 256;
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  kern<<<static_cast<unsigned>(grid), 128, smem, s>>>(mq, mk, p);
  KFA_CUDA(cudaGetLastError());
  return KFA_OK;
}

}  // namespace

extern "C" int kfa_scores(const KfaTensor4* q, const KfaTensor4* k, float* scores, int dtype, int* dev_status,
                          void* stream) {
  int rc;
  if ((rc = check_qkv(q, k, k, dtype, 0))) return rc;
  if (!scores || !dev_status) return fail(KFA_ERR_ARG, "scores / dev_status: null pointer");
  CUtensorMap mq, mk;
  if ((rc = make_map(q, dtype, &mq, "q")) || (rc = make_map(k, dtype, &mk, "k"))) return rc;
  kfa::ScoreParams p;
  p.out = scores;
  p.H = static_cast<int>(q->shape[1]);
  p.Sq = static_cast<int>(q->shape[2]);
  p.Skv = static_cast<int>(k->shape[2]);
  p.group = static_cast<int>(q->shape[1] / k->shape[1]);
  p.n_q128 = (p.Sq + 127) / 128;
  p.n_k128 = (p.Skv + 127) / 128;
  p.status = dev_status;
  const long long grid = static_cast<long long>(q->shape[0]) * p.H * p.n_q128 * p.n_k128;
  if (grid > 0x7fffffffll) return fail(KFA_ERR_ARG, "too many tiles");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(q->shape[3], dtype, (launch_scores<KD, KB>(mq, mk, p, grid, s)));
}
