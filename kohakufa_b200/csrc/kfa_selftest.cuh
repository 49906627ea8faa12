// kfa_selftest: one CTA exercises the building blocks of the attention kernels on small
// integer-valued matrices, where every product and sum is exact in fp16 / bf16 / fp32, and the
// host compares bit for bit:
//   1. TMA tile loads of two 128 x 128 16-bit matrices A, B (two 128B-swizzled 64-column boxes each)
//   2. S = A B^T      : both operands K-major in shared memory              -> out1 [128,128] fp32
//   3. P = 16-bit(S) stored to tensor memory, O = P B : A operand from tensor memory, B operand
//      MN-major in shared memory spanning two 64-column blocks                -> out2 [128,128] fp32
// Included at the end of kfa_api.cu (uses its helpers).
#pragma once

namespace kfa {

template <bool BF16>
__global__ void __launch_bounds__(128, 1)
kfa_selftest_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    float* out1, float* out2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sA = smem_base, sB = smem_base + 2 * TILE_BYTES_64;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 4 * TILE_BYTES_64);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const uint32_t bar0 = smem_u32(bars);
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(bar0 + 8 * i, 1);
    *s_abort = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(s_tmem), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const Ctl ctl{s_abort, status};
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  bool ok = true;

  if (tid == 0) {
    mbar_expect_tx(bar0, 4 * TILE_BYTES_64);
    for (int ch = 0; ch < 2; ++ch) {
      tma_load_4d(sA + ch * TILE_BYTES_64, &tmA, bar0, ch * 64, 0, 0, 0);
      tma_load_4d(sB + ch * TILE_BYTES_64, &tmB, bar0, ch * 64, 0, 0, 0);
    }
    ok = mbar_wait(bar0, 0, ctl, 91);
    if (ok) {
      tc_fence_after();
      constexpr uint32_t IDESC = make_idesc(BF16, false, 128, 128);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * TILE_BYTES_64 + (kk & 3) * 32;
        umma_ss(tmem, make_sdesc(sA + off, 16, 1024), make_sdesc(sB + off, 16, 1024), IDESC, kk > 0);
      }
      umma_commit(bar0 + 8);
    } else {
      mbar_drain(bar0, 0);  // gave up: the copies still have to land before the CTA leaves
    }
  }
  ok = mbar_wait_warp(bar0 + 8, 0, ctl, 92);
  if (ok) {
    tc_fence_after();
    float s[128];
    for (int g = 0; g < 4; ++g) tmem_ld32(tmem + lane_base + 32 * g, reinterpret_cast<uint32_t*>(s + 32 * g));
    tmem_wait_ld();
    for (int i = 0; i < 128; ++i) out1[tid * 128 + i] = s[i];
    for (int g = 0; g < 4; ++g) {
      uint32_t pk[16];
      for (int i = 0; i < 32; i += 2) pk[i / 2] = pack16<BF16>(s[32 * g + i], s[32 * g + i + 1]);
      tmem_st16(tmem + lane_base + 16 * g, pk);
    }
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && !*s_abort) {
    tc_fence_after();
    constexpr uint32_t IDESC = make_idesc(BF16, true, 128, 128);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      umma_ts(tmem + 128, tmem + kk * 8, make_sdesc(sB + kk * 2048, TILE_BYTES_64, 1024), IDESC, kk > 0);
    umma_commit(bar0 + 16);
  }
  ok = mbar_wait_warp(bar0 + 16, 0, ctl, 93);
  if (ok) {
    tc_fence_after();
    float o[128];
    for (int g = 0; g < 4; ++g) tmem_ld32(tmem + 128 + lane_base + 32 * g, reinterpret_cast<uint32_t*>(o + 32 * g));
    tmem_wait_ld();
    for (int i = 0; i < 128; ++i) out2[tid * 128 + i] = o[i];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

}  // namespace kfa

namespace {

template <bool BF16>
int selftest_one(std::string& rep) {
  const int N = 128;
  std::vector<uint16_t> hA(N * N), hB(N * N);
  std::vector<int> iA(N * N), iB(N * N);
  uint32_t lcg = BF16 ? 12345u : 54321u;
  auto next = [&]() {
    lcg = lcg * 1664525u + 1013904223u;
    return static_cast<int>((lcg >> 16) % 3) - 1;  // -1, 0, 1
  };
  auto enc = [&](int v) -> uint16_t {  // -1, 0, 1 in fp16 / bf16
    if (v == 0) return 0;
    const uint16_t one = BF16 ? 0x3F80 : 0x3C00;
    return v > 0 ? one : static_cast<uint16_t>(one | 0x8000);
  };
  for (int i = 0; i < N * N; ++i) {
    iA[i] = next();
    iB[i] = next();
    hA[i] = enc(iA[i]);
    hB[i] = enc(iB[i]);
  }
  std::vector<float> e1(N * N), e2(N * N);
  for (int i = 0; i < N; ++i)
    for (int j = 0; j < N; ++j) {
      int acc = 0;
      for (int k = 0; k < N; ++k) acc += iA[i * N + k] * iB[j * N + k];
      e1[i * N + j] = static_cast<float>(acc);
    }
  for (int i = 0; i < N; ++i)
    for (int d = 0; d < N; ++d) {
      int acc = 0;
      for (int j = 0; j < N; ++j) acc += static_cast<int>(e1[i * N + j]) * iB[j * N + d];
      e2[i * N + d] = static_cast<float>(acc);
    }

  uint16_t *dA = nullptr, *dB = nullptr;
  float *d1 = nullptr, *d2 = nullptr;
  int* dst = nullptr;
  auto cleanup = [&]() {
    cudaFree(dA);
    cudaFree(dB);
    cudaFree(d1);
    cudaFree(d2);
    cudaFree(dst);
  };
#define KFA_ST(expr)                                                                      \
  do {                                                                                    \
    cudaError_t e_ = (expr);                                                              \
    if (e_ != cudaSuccess) {                                                              \
      cleanup();                                                                          \
      return fail(KFA_ERR_CUDA, "selftest %s: %s", #expr, cudaGetErrorString(e_));        \
    }                                                                                     \
  } while (0)
  KFA_ST(cudaMalloc(&dA, N * N * 2));
  KFA_ST(cudaMalloc(&dB, N * N * 2));
  KFA_ST(cudaMalloc(&d1, N * N * 4));
  KFA_ST(cudaMalloc(&d2, N * N * 4));
  KFA_ST(cudaMalloc(&dst, 4));
  KFA_ST(cudaMemcpy(dA, hA.data(), N * N * 2, cudaMemcpyHostToDevice));
  KFA_ST(cudaMemcpy(dB, hB.data(), N * N * 2, cudaMemcpyHostToDevice));
  KFA_ST(cudaMemset(d1, 0xff, N * N * 4));
  KFA_ST(cudaMemset(d2, 0xff, N * N * 4));
  KFA_ST(cudaMemset(dst, 0, 4));
  KfaTensor4 tA{dA, {1, 1, N, N}, {N * N, N * N, N, 1}};
  KfaTensor4 tB{dB, {1, 1, N, N}, {N * N, N * N, N, 1}};
  CUtensorMap mA, mB;
  int rc;
  if ((rc = make_map(&tA, BF16 ? KFA_BF16 : KFA_F16, &mA, "A")) || (rc = make_map(&tB, BF16 ? KFA_BF16 : KFA_F16, &mB, "B"))) {
    cleanup();
    return rc;
  }
  const int smem = 4 * kfa::TILE_BYTES_64 + 1024 + 256;
  auto kern = kfa::kfa_selftest_kernel<BF16>;
  KFA_ST(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<1, 128, smem>>>(mA, mB, d1, d2, dst);
  KFA_ST(cudaGetLastError());
  KFA_ST(cudaDeviceSynchronize());
  std::vector<float> g1(N * N), g2(N * N);
  int hst = 0;
  KFA_ST(cudaMemcpy(g1.data(), d1, N * N * 4, cudaMemcpyDeviceToHost));
  KFA_ST(cudaMemcpy(g2.data(), d2, N * N * 4, cudaMemcpyDeviceToHost));
  KFA_ST(cudaMemcpy(&hst, dst, 4, cudaMemcpyDeviceToHost));
  cleanup();
#undef KFA_ST
  auto cmp = [&](const std::vector<float>& g, const std::vector<float>& e, const char* what) {
    int bad = 0, first = -1;
    for (int i = 0; i < N * N; ++i)
      if (!(g[i] == e[i])) {
        if (first < 0) first = i;
        ++bad;
      }
    char line[256];
    if (bad)
      snprintf(line, sizeof(line), "%s %s: %d / %d differ; first at [%d,%d]: got %g want %g\n", BF16 ? "bf16" : "fp16",
               what, bad, N * N, first / N, first % N, g[first], e[first]);
    else
      snprintf(line, sizeof(line), "%s %s: exact\n", BF16 ? "bf16" : "fp16", what);
    rep += line;
    return bad;
  };
  char line[64];
  snprintf(line, sizeof(line), "%s device status: %d\n", BF16 ? "bf16" : "fp16", hst);
  rep += line;
  const int bad = cmp(g1, e1, "S = A B^T (smem x smem, K-major)") + cmp(g2, e2, "O = P B (tmem x smem, MN-major)");
  return (bad || hst) ? KFA_ERR_SELFTEST : KFA_OK;
}

}  // namespace

namespace kfa {

// The fragment-shaped TMEM accesses of the dK / dV kernel against the one-lane-per-thread shape:
// a pattern stored with st.32x32b is read back with ld.16x256b.x8, and a pattern stored with
// st.16x128b.x8 / .x4 is read back with ld.32x32b. The host checks the documented element maps.
__global__ void __launch_bounds__(128, 1) kfa_selftest_frag_kernel(uint32_t* out_ld, uint32_t* out_st) {
  __shared__ uint32_t s_tmem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (warp == 0) {
    tmem_alloc(smem_u32(&s_tmem), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  uint32_t v[32];
  for (int c0 = 0; c0 < 64; c0 += 32) {  // lane = tid, columns 0..63: value = lane * 1000 + column
    for (int i = 0; i < 32; ++i) v[i] = tid * 1000 + c0 + i;
    tmem_st32(tmem + lane_base + c0, v);
  }
  tmem_wait_st();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  for (int half = 0; half < 2; ++half) {
    tmem_ld_16x256b_x8(tmem + lane_base + (static_cast<uint32_t>(16 * half) << 16), v);
    tmem_wait_ld();
    for (int i = 0; i < 32; ++i) out_ld[((warp * 2 + half) * 32 + lane) * 32 + i] = v[i];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  for (int half = 0; half < 2; ++half) {  // columns 64..95 by one x8 store, 96..127 by two x4 stores
    uint32_t w[16];
    for (int i = 0; i < 16; ++i) w[i] = (half << 16) | (lane << 8) | i;
    const uint32_t base = tmem + lane_base + (static_cast<uint32_t>(16 * half) << 16);
    tmem_st_16x128b_x8(base + 64, w);
    tmem_st_16x128b_x4(base + 96, w);
    tmem_st_16x128b_x4(base + 112, w + 8);
  }
  tmem_wait_st();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  for (int c0 = 64; c0 < 128; c0 += 32) {
    tmem_ld32(tmem + lane_base + c0, v);
    tmem_wait_ld();
    for (int i = 0; i < 32; ++i) out_st[tid * 64 + (c0 - 64) + i] = v[i];
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

int selftest_frag(std::string& rep) {
  uint32_t *d_ld = nullptr, *d_st = nullptr;
  const size_t n_ld = 4 * 2 * 32 * 32, n_st = 128 * 64;
  if (cudaMalloc(&d_ld, n_ld * 4) != cudaSuccess || cudaMalloc(&d_st, n_st * 4) != cudaSuccess) {
    cudaFree(d_ld);
    return fail(KFA_ERR_CUDA, "selftest: cudaMalloc failed");
  }
  kfa::kfa_selftest_frag_kernel<<<1, 128>>>(d_ld, d_st);
  std::vector<uint32_t> h_ld(n_ld), h_st(n_st);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(h_ld.data(), d_ld, n_ld * 4, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(h_st.data(), d_st, n_st * 4, cudaMemcpyDeviceToHost);
  cudaFree(d_ld);
  cudaFree(d_st);
  if (e != cudaSuccess) return fail(KFA_ERR_CUDA, "selftest fragments: %s", cudaGetErrorString(e));
  int bad_ld = 0, bad_st = 0;
  // ld.16x256b.x8: r[4j + q] = (lane l/4 + 8 (q >= 2), column 8j + 2 (l % 4) + (q & 1))
  for (int w = 0; w < 4; ++w)
    for (int half = 0; half < 2; ++half)
      for (int l = 0; l < 32; ++l)
        for (int i = 0; i < 32; ++i) {
          const int j = i / 4, q = i % 4;
          const uint32_t row = w * 32 + half * 16 + l / 4 + (q >= 2 ? 8 : 0), col = 8 * j + 2 * (l % 4) + (q & 1);
          bad_ld += h_ld[((w * 2 + half) * 32 + l) * 32 + i] != row * 1000 + col;
        }
  // st.16x128b: r[2j + s] -> (lane l/4 + 8 s, column 4j + l % 4), columns counted from the store's address
  for (int t = 0; t < 128; ++t)
    for (int c = 0; c < 64; ++c) {
      const int half = (t % 32) / 16, r16 = t % 16;
      const int cc = c < 32 ? c : (c < 48 ? c - 32 : c - 48);  // column inside its store
      const int reg0 = c < 32 ? 0 : (c < 48 ? 0 : 8);          // first register of its store
      const uint32_t want = (half << 16) | (((r16 % 8) * 4 + cc % 4) << 8) | (reg0 + 2 * (cc / 4) + (r16 >= 8 ? 1 : 0));
      bad_st += h_st[t * 64 + c] != want;
    }
  char line[160];
  snprintf(line, sizeof(line), "tmem fragments: ld.16x256b %s, st.16x128b %s\n", bad_ld ? "differ" : "exact",
           bad_st ? "differ" : "exact");
  rep += line;
  return (bad_ld || bad_st) ? KFA_ERR_SELFTEST : KFA_OK;
}

}  // namespace

extern "C" int kfa_selftest(char* report, int report_len) {
  std::string rep;
  const int r1 = selftest_one<false>(rep);
  int r2 = (r1 == KFA_ERR_CUDA) ? r1 : selftest_one<true>(rep);
  if (r2 != KFA_ERR_CUDA) {
    const int r3 = selftest_frag(rep);
    if (r3) r2 = r3;
  }
  if (report && report_len > 0) {
    std::strncpy(report, rep.c_str(), report_len - 1);
    report[report_len - 1] = 0;
  }
  if (r1 == KFA_ERR_CUDA || r2 == KFA_ERR_CUDA) return KFA_ERR_CUDA;
  if (r1 || r2) return fail(KFA_ERR_SELFTEST, "selftest mismatch:\n%s", rep.c_str());
  return KFA_OK;
}
