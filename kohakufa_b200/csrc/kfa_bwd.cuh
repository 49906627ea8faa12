// Attention backward for sm_100a, as three kernels:
//
//   kfa_bwd_prepare_kernel   delta = rowsum(fp32(dO) * fp32(O)); packs (m, log2 l, delta) per
//                            128-row query tile, padded rows get m = +inf so their P is 0
//                            (reference: src/kohakufa/sm100/bwd.py:1358-1388)
//   kfa_bwd_dkdv_kernel      one CTA per (batch, head, 128-key tile), looping over the query
//                            tiles that see it, everything transposed (keys on TMEM lanes):
//                              S^T = K Q_i^T, dP^T = V dO_i^T, dV += P^T dO_i, dK += dS^T Q_i
//                            (reference: bwd.py:565-694 MMAs, 967-1127 P / dS partitions)
//   kfa_bwd_dq_kernel        one CTA per (batch, head, 128-query tile), looping over key tiles:
//                              S = Q K_j^T, dP = dO V_j^T, dQ += dS K_j
//
// The reference fuses dQ into the key-major kernel and accumulates it with fp32 reduce-adds into
// a scratch buffer (bwd.py:1135-1232, 1391-1410). Here dQ has its own query-major kernel: two more
// MMAs per tile pair, but no atomics, no fp32 accumulator round trip through HBM, and dQ is
// bit-reproducible run to run.
//
// Both main kernels split every 128x128 score tile into two 64-column halves (a, b), each owned
// by one warpgroup, so the tensor core works on one half while the warpgroup of the other half
// computes P and dS:
//   warps 0-3  half a        warps 4-7  half b        warp 8  MMA issue        warp 9  TMA producer
// P^T / dS^T (dS in the dQ kernel) are written 16-bit into TMEM over the S / dP columns they came
// from and are consumed from there as the A operand of the following MMAs.
//
// Numerics kept from the reference (docs/precision.md:27-34, 90-114; bwd.py:1036-1043, 1083-1086):
//   * P = exp2(fma(S - m, c, -log2 l)) from the two separate statistics, never a fused lse;
//   * dS = (dP - delta) * P16 with P16 the 16-bit rounded P; dS, not scale * dS, is rounded to
//     16 bits and fed to the MMAs; scale multiplies the fp32 dK and dQ accumulators afterwards;
//   * padded keys and hidden (key, query) pairs get P = 0 exactly; padded query rows carry m = +inf.
#pragma once

#include "kfa_fwd.cuh"

namespace kfa {

struct BwdParams {
  void* dq;  // [B, H, Sq, D] view
  long long dq_sb, dq_sh, dq_ss;
  void* dk;  // [B, H, Skv, D] view
  long long dk_sb, dk_sh, dk_ss;
  void* dv;
  long long dv_sb, dv_sh, dv_ss;
  const float* stats;  // [B*H, n_q128, 3, 128]: m, log2 l, delta
  int B, H, Sq, Skv;
  int P;
  float c;      // scale * log2(e)
  float scale;  // applied to fp32 dK and dQ
  int n_q128, n_k128;
  int* status;
};

struct PrepParams {
  const void* o;
  long long o_sb, o_sh, o_ss;
  const void* dout;
  long long do_sb, do_sh, do_ss;
  const float* lse;  // [B, H, 2, Sq]
  float* stats;      // [B*H, n_q128, 3, 128]
  int B, H, Sq, n_q128;
};

// ---------------------------------------------------------------------------------------
// prepare: HBM-bound; D / 8 lanes per row, 16-byte loads.
// ---------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(128) kfa_bwd_prepare_kernel(const PrepParams p) {
  constexpr int LPR = D / 8;       // lanes per row
  constexpr int RPW = 32 / LPR;    // rows per warp pass
  const int tile = blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, vec = lane % LPR;
  const uint8_t* ob = reinterpret_cast<const uint8_t*>(p.o) + 2 * (b * p.o_sb + h * p.o_sh);
  const uint8_t* gb = reinterpret_cast<const uint8_t*>(p.dout) + 2 * (b * p.do_sb + h * p.do_sh);
  float* st = p.stats + (static_cast<long long>(bh) * p.n_q128 + tile) * 384;
  const float* lse = p.lse + static_cast<long long>(bh) * 2 * p.Sq;
  for (int r0 = warp * 32; r0 < warp * 32 + 32; r0 += RPW) {
    const int r_in = r0 + sub;
    const int row = tile * 128 + r_in;
    float acc = 0.f;
    if (row < p.Sq) {
      const uint4 ov = *reinterpret_cast<const uint4*>(ob + 2 * (row * p.o_ss + vec * 8));
      const uint4 gv = *reinterpret_cast<const uint4*>(gb + 2 * (row * p.do_ss + vec * 8));
      const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = unpack16<BF16>(ow[i]);
        const float2 g = unpack16<BF16>(gw[i]);
        acc = fmaf(a.x, g.x, acc);
        acc = fmaf(a.y, g.y, acc);
      }
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (vec == 0) {
      const bool valid = row < p.Sq;
      // stored negated, so the consumers only add; padded rows: -m = -inf makes their P exactly 0
      st[r_in] = valid ? -lse[row] : -INFINITY;
      st[128 + r_in] = valid ? -lse[p.Sq + row] : 0.f;
      st[256 + r_in] = valid ? -acc : 0.f;
    }
  }
}

// ---------------------------------------------------------------------------------------
// shared configuration of the two main kernels
// ---------------------------------------------------------------------------------------
constexpr int BWD_THREADS = 320;
constexpr int STATS_BYTES = 3 * 128 * 4;

template <int D>
struct BwdCfg {
  static constexpr int CHUNKS = D / 64;
  static constexpr int TILE_BYTES = CHUNKS * TILE_BYTES_64;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t TM_S = 0, TM_DP = 128, TM_ACC0 = 256, TM_ACC1 = 256 + D;
  // dK/dV kernel: K, V resident; ring of (Q_i, dO_i, stats_i) slots.
  static constexpr int KV_SLOTS = (D == 128) ? 2 : 3;
  static constexpr int KV_SLOT_BYTES = 2 * TILE_BYTES + 2048;  // stats padded to keep 1 KB alignment
  static constexpr int KV_SMEM_TILES = 2 * TILE_BYTES + KV_SLOTS * KV_SLOT_BYTES;
  static constexpr int KV_SMEM_BYTES = KV_SMEM_TILES + 1024 + 256;
  // dQ kernel: Q, dO resident; ring of (K_j, V_j) slots.
  static constexpr int Q_SLOTS = (D == 128) ? 2 : 3;
  static constexpr int Q_SLOT_BYTES = 2 * TILE_BYTES;
  static constexpr int Q_SMEM_TILES = 2 * TILE_BYTES + Q_SLOTS * Q_SLOT_BYTES;
  static constexpr int Q_SMEM_BYTES = Q_SMEM_TILES + 1024 + 256;
};

// Issue helpers for the MMA warp (converged; `lead` is true in the one lane that issues). Operand
// tiles are 128B-swizzled [rows][64] boxes, D / 64 of them 16 KB apart; descriptors are passed as
// their low words (see sdesc_lo).
// acc[128 x 64] = A[128 rows, D] * B[64 rows, D]^T, contraction over D. b_lo already points at B's
// first row.
template <int D>
__device__ __forceinline__ void issue_kmajor_n64(bool lead, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                 uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const uint32_t off = ((kk >> 2) * TILE_BYTES_64 + (kk & 3) * 32) >> 4;
    umma_ss_lead(lead, d_tmem, a_lo + off, b_lo + off, idesc, kk > 0 ? 1u : 0u);
  }
}
// acc[128 x D] (+)= A16[128 x 64 from TMEM] * B[64 rows, D], contraction over B's rows (MN-major B,
// leading offset = one 16 KB box). b_lo points at B's first row.
template <int D>
__device__ __forceinline__ void issue_tmemA_k64(bool lead, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                                uint32_t idesc, bool acc) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    umma_ts_lead(lead, d_tmem, a_tmem + kk * 8, b_lo + ((kk * 16 * 128) >> 4), idesc, (acc || kk > 0) ? 1u : 0u);
}

// Writes a row of an fp32 accumulator (TMEM columns [col0, col0 + ncols)) times mul as 16-bit.
template <bool BF16>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, int col0, int ncols, float mul, uint8_t* grow,
                                              bool valid) {
  for (int cc = col0; cc < col0 + ncols; cc += 32) {
    float o[32];
    tmem_ld32(taddr + cc, reinterpret_cast<uint32_t*>(o));
    tmem_wait_ld();
    if (valid) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 w;
        w.x = pack16<BF16>(o[i] * mul, o[i + 1] * mul);
        w.y = pack16<BF16>(o[i + 2] * mul, o[i + 3] * mul);
        w.z = pack16<BF16>(o[i + 4] * mul, o[i + 5] * mul);
        w.w = pack16<BF16>(o[i + 6] * mul, o[i + 7] * mul);
        *reinterpret_cast<uint4*>(grow + 2 * (cc + i)) = w;
      }
    }
  }
}

// 32 columns (queries) of one key row in the dK / dV kernel: from S^T and dP^T (fp32, two columns
// per float2) and the per-query statistics in shared memory (-m at st[0..], -log2 l at st[128..],
// -delta at st[256..]) to the packed 16-bit P^T and dS^T words.
//   P = exp2(fma(S - m, c, -log2 l));  dS = (dP - delta) * P   (fp32 P; dS rounded once, unscaled)
// MASKED: columns whose query index (q_first + column) is below qmin get P = dS = 0.
template <bool BF16, bool MASKED>
__device__ __forceinline__ void pds_cols_by_query(const float2* sv, const float2* dp, const float* st, float2 c2,
                                                  int q_first, int qmin, uint32_t* pk, uint32_t* dk) {
#pragma unroll
  for (int x = 0; x < 32; x += 4) {
    const float4 nm = *reinterpret_cast<const float4*>(st + x);
    const float4 nl = *reinterpret_cast<const float4*>(st + 128 + x);
    const float4 nd = *reinterpret_cast<const float4*>(st + 256 + x);
    const float2 x0 = __ffma2_rn(__fadd2_rn(sv[x / 2], make_float2(nm.x, nm.y)), c2, make_float2(nl.x, nl.y));
    const float2 x1 = __ffma2_rn(__fadd2_rn(sv[x / 2 + 1], make_float2(nm.z, nm.w)), c2, make_float2(nl.z, nl.w));
    float2 p0 = make_float2(ex2(x0.x), ex2(x0.y));
    float2 p1 = make_float2(ex2(x1.x), ex2(x1.y));
    if constexpr (MASKED) {
      if (q_first + x < qmin) p0.x = 0.f;
      if (q_first + x + 1 < qmin) p0.y = 0.f;
      if (q_first + x + 2 < qmin) p1.x = 0.f;
      if (q_first + x + 3 < qmin) p1.y = 0.f;
    }
    pk[x / 2] = pack16<BF16>(p0.x, p0.y);
    pk[x / 2 + 1] = pack16<BF16>(p1.x, p1.y);
    const float2 d0 = __fmul2_rn(__fadd2_rn(dp[x / 2], make_float2(nd.x, nd.y)), p0);
    const float2 d1 = __fmul2_rn(__fadd2_rn(dp[x / 2 + 1], make_float2(nd.z, nd.w)), p1);
    dk[x / 2] = pack16<BF16>(d0.x, d0.y);
    dk[x / 2 + 1] = pack16<BF16>(d1.x, d1.y);
  }
}

// 32 columns (keys) of one query row in the dQ kernel: the row's statistics are scalars.
// MASKED: columns at or beyond `lim` (relative to this group's first column) get dS = 0.
template <bool BF16, bool MASKED>
__device__ __forceinline__ void ds_cols_by_key(const float2* sv, const float2* dp, float2 nm, float2 c2, float2 nl,
                                               float2 nd, int lim, uint32_t* dk) {
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    const float2 e = __ffma2_rn(__fadd2_rn(sv[x], nm), c2, nl);
    float2 pr = make_float2(ex2(e.x), ex2(e.y));
    if constexpr (MASKED) {
      if (2 * x >= lim) pr.x = 0.f;
      if (2 * x + 1 >= lim) pr.y = 0.f;
    }
    const float2 d = __fmul2_rn(__fadd2_rn(dp[x], nd), pr);
    dk[x] = pack16<BF16>(d.x, d.y);
  }
}

// ---------------------------------------------------------------------------------------
// dK / dV
// ---------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(BWD_THREADS, 1)
kfa_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const BwdParams p) {
  using Cfg = BwdCfg<D>;
  constexpr int CH = Cfg::CHUNKS;
  constexpr int NSL = Cfg::KV_SLOTS;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sK = smem_base;
  const uint32_t sV = smem_base + Cfg::TILE_BYTES;
  const uint32_t sSlot = smem_base + 2 * Cfg::TILE_BYTES;  // slot: Q | dO | stats
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::KV_SMEM_TILES);
  constexpr int B_KV = 0;                 // 1
  constexpr int B_QREADY = 1;             // NSL
  constexpr int B_QFREE = 1 + NSL;        // NSL
  constexpr int B_SDP = 1 + 2 * NSL;      // 2
  constexpr int B_PDS = 3 + 2 * NSL;      // 2
  constexpr int B_ACC = 5 + 2 * NSL;      // 1
  constexpr int B_DRAIN = 6 + 2 * NSL;    // 1
  constexpr int N_BARS = 7 + 2 * NSL;
  static_assert(N_BARS * 8 + 16 <= 256, "barrier block too small");
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // tile decode: head-major; when causal the first key tiles see the most queries and come first
  const int bh = blockIdx.x / p.n_k128;
  const int kt = blockIdx.x % p.n_k128;
  const int b = bh / p.H, h = bh % p.H;
  const int kv0 = kt * 128;
  const int first_i = (p.P > 0) ? static_cast<int>((static_cast<long long>(kv0 / p.P) * p.P) / 128) : 0;
  const int n_steps = max(p.n_q128 - first_i, 0);
  const bool ragged_keys = kv0 + 128 > p.Skv;

  if (tid == 0) {
    mbar_init(bar(B_KV), 1);
    for (int i = 0; i < NSL; ++i) {
      mbar_init(bar(B_QREADY + i), 1);
      mbar_init(bar(B_QFREE + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_SDP + i), 1);
      mbar_init(bar(B_PDS + i), 128);
    }
    mbar_init(bar(B_ACC), 1);
    mbar_init(bar(B_DRAIN), 1);
    *s_abort = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(s_tmem), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
#ifdef KFA_PROFILE
  long long prof_acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  long long kfa_prof_tb = 0;
  (void)kfa_prof_tb;
  const long long prof_t0 = clock64();
  const Ctl ctl{s_abort, p.status, prof_acc};
#else
  const Ctl ctl{s_abort, p.status};
#endif
  const bool dead = (*s_abort != 0);

  if (dead) {
  } else if (warp == 9) {
    // =========================== TMA producer ===========================
    if (lane == 0 && n_steps > 0) {
      prefetch_tensormap(&tmQ);
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmV);
      prefetch_tensormap(&tmDO);
      mbar_expect_tx(bar(B_KV), 2 * Cfg::TILE_BYTES);
      for (int ch = 0; ch < CH; ++ch) {
        tma_load_4d(sK + ch * TILE_BYTES_64, &tmK, bar(B_KV), ch * 64, kv0, h, b);
        tma_load_4d(sV + ch * TILE_BYTES_64, &tmV, bar(B_KV), ch * 64, kv0, h, b);
      }
      bool ok = true;
      int issued = 0;
      for (int s = 0; s < n_steps; ++s) {
        const int slot = s % NSL, use = s / NSL;
        if (use > 0) ok = mbar_wait(bar(B_QFREE + slot), (use - 1) & 1, ctl, 11);
        if (!ok) break;
        const int i = first_i + s;
        const uint32_t base = sSlot + slot * Cfg::KV_SLOT_BYTES;
        mbar_expect_tx(bar(B_QREADY + slot), 2 * Cfg::TILE_BYTES + STATS_BYTES);
        for (int ch = 0; ch < CH; ++ch) {
          tma_load_4d(base + ch * TILE_BYTES_64, &tmQ, bar(B_QREADY + slot), ch * 64, i * 128, h, b);
          tma_load_4d(base + Cfg::TILE_BYTES + ch * TILE_BYTES_64, &tmDO, bar(B_QREADY + slot), ch * 64,
                      i * 128, h, b);
        }
        bulk_load(base + 2 * Cfg::TILE_BYTES, p.stats + (static_cast<long long>(bh) * p.n_q128 + i) * 384,
                  STATS_BYTES, bar(B_QREADY + slot));
        issued = s + 1;
      }
      if (!ok) {
        for (int s = max(issued - NSL, 0); s < issued; ++s) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar(B_QREADY + s % NSL), (s / NSL) & 1) && clock64() - t0 < 2000000ll) {
          }
        }
      }
    }
  } else if (warp == 8) {
    // =========================== MMA issue ===========================
    // The whole warp runs this role converged; one elected lane issues the tcgen05 instructions.
    if (n_steps > 0) {
      const bool lead = elect_one();
      constexpr uint32_t IDESC_S = make_idesc(BF16, false, 128, 64);
      constexpr uint32_t IDESC_ACC = make_idesc(BF16, true, 128, D);
      const uint32_t tST = tmem + Cfg::TM_S, tDP = tmem + Cfg::TM_DP;
      const uint32_t tDV = tmem + Cfg::TM_ACC0, tDK = tmem + Cfg::TM_ACC1;
      const uint32_t k_lo = sdesc_lo(sK, 16), v_lo = sdesc_lo(sV, 16);
      constexpr uint32_t HALF_ROWS = (64 * 128) >> 4;  // 64 rows further down a box, in descriptor units
      bool ok = mbar_wait_warp(bar(B_KV), 0, ctl, 12);
      if (ok) ok = mbar_wait_warp(bar(B_QREADY + 0), 0, ctl, 13);
      if (ok) {
        tc_fence_after();
        const uint32_t q_lo = sdesc_lo(sSlot, 16), do_lo = sdesc_lo(sSlot + Cfg::TILE_BYTES, 16);
        for (int hq = 0; hq < 2; ++hq) {
          issue_kmajor_n64<D>(lead, tST + 64 * hq, k_lo, q_lo + hq * HALF_ROWS, IDESC_S);
          issue_kmajor_n64<D>(lead, tDP + 64 * hq, v_lo, do_lo + hq * HALF_ROWS, IDESC_S);
          umma_commit_lead(lead, bar(B_SDP + hq));
        }
      }
      for (int s = 0; s < n_steps && ok; ++s) {
        const int slot = s % NSL;
        const uint32_t q_s = sSlot + slot * Cfg::KV_SLOT_BYTES;
        const uint32_t do_s = q_s + Cfg::TILE_BYTES;
        const int nslot = (s + 1) % NSL;
        const uint32_t q_n = sSlot + nslot * Cfg::KV_SLOT_BYTES;
        const uint32_t do_n = q_n + Cfg::TILE_BYTES;
        // as the MN-major B operand of dV / dK (leading offset: the next 64 columns of D)
        const uint32_t qmn_lo = sdesc_lo(q_s, TILE_BYTES_64), domn_lo = sdesc_lo(do_s, TILE_BYTES_64);
        // as the K-major B operand of the next step's S^T / dP^T
        const uint32_t qn_lo = sdesc_lo(q_n, 16), don_lo = sdesc_lo(do_n, 16);
        for (int hq = 0; hq < 2 && ok; ++hq) {
          ok = mbar_wait_warp(bar(B_PDS + hq), s & 1, ctl, 14);
          if (!ok) break;
          tc_fence_after();
          issue_tmemA_k64<D>(lead, tDV, tST + 64 * hq, domn_lo + hq * HALF_ROWS, IDESC_ACC, s > 0 || hq > 0);
          issue_tmemA_k64<D>(lead, tDK, tDP + 64 * hq, qmn_lo + hq * HALF_ROWS, IDESC_ACC, s > 0 || hq > 0);
          if (hq == 1) umma_commit_lead(lead, bar(B_QFREE + slot));
          if (s + 1 < n_steps) {
            if (hq == 0) {
              ok = mbar_wait_warp(bar(B_QREADY + nslot), ((s + 1) / NSL) & 1, ctl, 15);
              if (!ok) break;
              tc_fence_after();
            }
            issue_kmajor_n64<D>(lead, tST + 64 * hq, k_lo, qn_lo + hq * HALF_ROWS, IDESC_S);
            issue_kmajor_n64<D>(lead, tDP + 64 * hq, v_lo, don_lo + hq * HALF_ROWS, IDESC_S);
            umma_commit_lead(lead, bar(B_SDP + hq));
          }
        }
      }
      if (ok) umma_commit_lead(lead, bar(B_ACC));
      umma_commit_lead(lead, bar(B_DRAIN));
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(bar(B_DRAIN), 0) && clock64() - t0 < KFA_WAIT_CYCLES) {
        }
      }
    }
  } else {
    // =========================== P^T / dS^T and epilogue ===========================
    const int hq = warp >> 2;
    const int k_in = tid & 127;
    const int key = kv0 + k_in;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + Cfg::TM_S + 64 * hq + lane_base;
    const uint32_t tDP = tmem + Cfg::TM_DP + 64 * hq + lane_base;
    // first query that sees this key; padded keys see nothing
    int qmin = 0;
    if (key >= p.Skv) qmin = 0x7fffffff;
    else if (p.P > 0) qmin = (key / p.P) * p.P;
    const float c = p.c;
    bool ok = true;
    for (int s = 0; s < n_steps; ++s) {
      const int slot = s % NSL;
      const int i = first_i + s;
      const int q0 = i * 128 + 64 * hq;  // query of this half's column 0
      // masked step: some (key, query) pair of this tile pair is hidden, or keys are padded
      const bool masked = ragged_keys || (p.P > 0 && key_limit(i * 128, p.P, p.Skv) < kv0 + 128);
      ok = mbar_wait_warp(bar(B_QREADY + slot), (s / NSL) & 1, ctl, 16);  // stats of this step
      if (ok) ok = mbar_wait_warp(bar(B_SDP + hq), s & 1, ctl, 17);
      if (!ok) break;
      tc_fence_after();
      const float* st =
          reinterpret_cast<const float*>(smem + 2 * Cfg::TILE_BYTES + slot * Cfg::KV_SLOT_BYTES +
                                         2 * Cfg::TILE_BYTES) + 64 * hq;
      const float2 c2 = make_float2(c, c);
      {
        float2 sv[32], dp[32];  // 64 columns of S^T and of dP^T
        tmem_ld32(tS, reinterpret_cast<uint32_t*>(sv));
        tmem_ld32(tDP, reinterpret_cast<uint32_t*>(dp));
        tmem_ld32(tS + 32, reinterpret_cast<uint32_t*>(sv + 16));
        tmem_ld32(tDP + 32, reinterpret_cast<uint32_t*>(dp + 16));
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint32_t pk[16], dk[16];
          if (masked)
            pds_cols_by_query<BF16, true>(sv + 16 * g, dp + 16 * g, st + 32 * g, c2, q0 + 32 * g, qmin, pk, dk);
          else
            pds_cols_by_query<BF16, false>(sv + 16 * g, dp + 16 * g, st + 32 * g, c2, q0 + 32 * g, qmin, pk, dk);
          // 16-bit P^T / dS^T over columns already read
          tmem_st16(tS + 16 * g, pk);
          tmem_st16(tDP + 16 * g, dk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(B_PDS + hq));
    }
    // ---- epilogue: half a stores dV, half b stores scale * dK ----
    const bool valid = key < p.Skv;
    uint8_t* grow;
    if (hq == 0)
      grow = reinterpret_cast<uint8_t*>(p.dv) + 2 * (b * p.dv_sb + h * p.dv_sh + static_cast<long long>(key) * p.dv_ss);
    else
      grow = reinterpret_cast<uint8_t*>(p.dk) + 2 * (b * p.dk_sb + h * p.dk_sh + static_cast<long long>(key) * p.dk_ss);
    if (n_steps == 0) {
      if (valid)
        for (int cc = 0; cc < D; cc += 8) *reinterpret_cast<uint4*>(grow + 2 * cc) = make_uint4(0, 0, 0, 0);
    } else {
      ok = mbar_wait_warp(bar(B_ACC), 0, ctl, 18) && ok;
      if (ok) {
        tc_fence_after();
        store_acc_row<BF16>(tmem + (hq ? Cfg::TM_ACC1 : Cfg::TM_ACC0) + lane_base, 0, D,
                            hq ? p.scale : 1.0f, grow, valid);
      }
    }
  }

#ifdef KFA_PROFILE
  prof_acc[0] = clock64() - prof_t0;
  if (lane == 0 && (warp == 0 || warp == 4 || warp == 8 || warp == 9))
    kfa_prof_flush(prof_acc, warp == 0 ? 0 : (warp == 4 ? 1 : (warp == 8 ? 2 : 3)));
#endif
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// dQ
// ---------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(BWD_THREADS, 1)
kfa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                  const BwdParams p) {
  using Cfg = BwdCfg<D>;
  constexpr int CH = Cfg::CHUNKS;
  constexpr int NSL = Cfg::Q_SLOTS;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base;
  const uint32_t sDO = smem_base + Cfg::TILE_BYTES;
  const uint32_t sSlot = smem_base + 2 * Cfg::TILE_BYTES;  // slot: K | V
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::Q_SMEM_TILES);
  constexpr int B_Q = 0;
  constexpr int B_KVREADY = 1;
  constexpr int B_KVFREE = 1 + NSL;
  constexpr int B_SDP = 1 + 2 * NSL;
  constexpr int B_DS = 3 + 2 * NSL;
  constexpr int B_ACC = 5 + 2 * NSL;
  constexpr int B_DRAIN = 6 + 2 * NSL;
  constexpr int N_BARS = 7 + 2 * NSL;
  static_assert(N_BARS * 8 + 16 <= 256, "barrier block too small");
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int bh = blockIdx.x / p.n_q128;
  const int t = blockIdx.x % p.n_q128;
  const int qt = (p.P > 0) ? (p.n_q128 - 1 - t) : t;
  const int b = bh / p.H, h = bh % p.H;
  const int row0 = qt * 128;
  const int last = min(row0 + 127, p.Sq - 1);
  const int n_steps = (key_limit(last, p.P, p.Skv) + 127) / 128;
  const int n_unmasked = key_limit(row0, p.P, p.Skv) / 128;

  if (tid == 0) {
    mbar_init(bar(B_Q), 1);
    for (int i = 0; i < NSL; ++i) {
      mbar_init(bar(B_KVREADY + i), 1);
      mbar_init(bar(B_KVFREE + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_SDP + i), 1);
      mbar_init(bar(B_DS + i), 128);
    }
    mbar_init(bar(B_ACC), 1);
    mbar_init(bar(B_DRAIN), 1);
    *s_abort = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(s_tmem), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
#ifdef KFA_PROFILE
  long long prof_acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  long long kfa_prof_tb = 0;
  (void)kfa_prof_tb;
  const long long prof_t0 = clock64();
  const Ctl ctl{s_abort, p.status, prof_acc};
#else
  const Ctl ctl{s_abort, p.status};
#endif
  const bool dead = (*s_abort != 0);

  if (dead) {
  } else if (warp == 9) {
    if (lane == 0) {
      prefetch_tensormap(&tmQ);
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmV);
      prefetch_tensormap(&tmDO);
      mbar_expect_tx(bar(B_Q), 2 * Cfg::TILE_BYTES);
      for (int ch = 0; ch < CH; ++ch) {
        tma_load_4d(sQ + ch * TILE_BYTES_64, &tmQ, bar(B_Q), ch * 64, row0, h, b);
        tma_load_4d(sDO + ch * TILE_BYTES_64, &tmDO, bar(B_Q), ch * 64, row0, h, b);
      }
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_steps; ++j) {
        const int slot = j % NSL, use = j / NSL;
        if (use > 0) ok = mbar_wait(bar(B_KVFREE + slot), (use - 1) & 1, ctl, 21);
        if (!ok) break;
        const uint32_t base = sSlot + slot * Cfg::Q_SLOT_BYTES;
        mbar_expect_tx(bar(B_KVREADY + slot), 2 * Cfg::TILE_BYTES);
        for (int ch = 0; ch < CH; ++ch) {
          tma_load_4d(base + ch * TILE_BYTES_64, &tmK, bar(B_KVREADY + slot), ch * 64, j * 128, h, b);
          tma_load_4d(base + Cfg::TILE_BYTES + ch * TILE_BYTES_64, &tmV, bar(B_KVREADY + slot), ch * 64,
                      j * 128, h, b);
        }
        issued = j + 1;
      }
      if (!ok) {
        for (int j = max(issued - NSL, 0); j < issued; ++j) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar(B_KVREADY + j % NSL), (j / NSL) & 1) && clock64() - t0 < 2000000ll) {
          }
        }
      }
    }
  } else if (warp == 8) {
    // MMA issue: the whole warp converged, one elected lane issues.
    {
      const bool lead = elect_one();
      constexpr uint32_t IDESC_S = make_idesc(BF16, false, 128, 64);
      constexpr uint32_t IDESC_ACC = make_idesc(BF16, true, 128, D);
      const uint32_t tS = tmem + Cfg::TM_S, tDP = tmem + Cfg::TM_DP, tDQ = tmem + Cfg::TM_ACC0;
      const uint32_t q_lo = sdesc_lo(sQ, 16), do_lo = sdesc_lo(sDO, 16);
      constexpr uint32_t HALF_ROWS = (64 * 128) >> 4;
      bool ok = mbar_wait_warp(bar(B_Q), 0, ctl, 22);
      if (ok) ok = mbar_wait_warp(bar(B_KVREADY + 0), 0, ctl, 23);
      if (ok) {
        tc_fence_after();
        const uint32_t k_lo = sdesc_lo(sSlot, 16), v_lo = sdesc_lo(sSlot + Cfg::TILE_BYTES, 16);
        for (int hk = 0; hk < 2; ++hk) {
          issue_kmajor_n64<D>(lead, tS + 64 * hk, q_lo, k_lo + hk * HALF_ROWS, IDESC_S);
          issue_kmajor_n64<D>(lead, tDP + 64 * hk, do_lo, v_lo + hk * HALF_ROWS, IDESC_S);
          umma_commit_lead(lead, bar(B_SDP + hk));
        }
      }
      for (int j = 0; j < n_steps && ok; ++j) {
        const int slot = j % NSL;
        const uint32_t k_s = sSlot + slot * Cfg::Q_SLOT_BYTES;
        const int nslot = (j + 1) % NSL;
        const uint32_t k_n = sSlot + nslot * Cfg::Q_SLOT_BYTES;
        const uint32_t kmn_lo = sdesc_lo(k_s, TILE_BYTES_64);
        const uint32_t kn_lo = sdesc_lo(k_n, 16), vn_lo = sdesc_lo(k_n + Cfg::TILE_BYTES, 16);
        for (int hk = 0; hk < 2 && ok; ++hk) {
          ok = mbar_wait_warp(bar(B_DS + hk), j & 1, ctl, 24);
          if (!ok) break;
          tc_fence_after();
          issue_tmemA_k64<D>(lead, tDQ, tDP + 64 * hk, kmn_lo + hk * HALF_ROWS, IDESC_ACC, j > 0 || hk > 0);
          if (hk == 1) umma_commit_lead(lead, bar(B_KVFREE + slot));
          if (j + 1 < n_steps) {
            if (hk == 0) {
              ok = mbar_wait_warp(bar(B_KVREADY + nslot), ((j + 1) / NSL) & 1, ctl, 25);
              if (!ok) break;
              tc_fence_after();
            }
            issue_kmajor_n64<D>(lead, tS + 64 * hk, q_lo, kn_lo + hk * HALF_ROWS, IDESC_S);
            issue_kmajor_n64<D>(lead, tDP + 64 * hk, do_lo, vn_lo + hk * HALF_ROWS, IDESC_S);
            umma_commit_lead(lead, bar(B_SDP + hk));
          }
        }
      }
      if (ok) umma_commit_lead(lead, bar(B_ACC));
      umma_commit_lead(lead, bar(B_DRAIN));
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(bar(B_DRAIN), 0) && clock64() - t0 < KFA_WAIT_CYCLES) {
        }
      }
    }
  } else {
    const int hk = warp >> 2;
    const int r_in = tid & 127;
    const int row = row0 + r_in;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + Cfg::TM_S + 64 * hk + lane_base;
    const uint32_t tDP = tmem + Cfg::TM_DP + 64 * hk + lane_base;
    const float* st = p.stats + (static_cast<long long>(bh) * p.n_q128 + qt) * 384;
    const float2 nm = make_float2(st[r_in], st[r_in]);                // -m
    const float2 nl = make_float2(st[128 + r_in], st[128 + r_in]);    // -log2 l
    const float2 nd = make_float2(st[256 + r_in], st[256 + r_in]);    // -delta
    const int my_limit = key_limit(min(row, p.Sq - 1), p.P, p.Skv);
    const float2 c2 = make_float2(p.c, p.c);
    bool ok = true;
    for (int j = 0; j < n_steps; ++j) {
      ok = mbar_wait_warp(bar(B_SDP + hk), j & 1, ctl, 26);
      if (!ok) break;
      tc_fence_after();
      const int lim = my_limit - j * 128 - 64 * hk;  // visible columns of this half (masked tiles)
      {
        float2 sv[32], dp[32];
        tmem_ld32(tS, reinterpret_cast<uint32_t*>(sv));
        tmem_ld32(tDP, reinterpret_cast<uint32_t*>(dp));
        tmem_ld32(tS + 32, reinterpret_cast<uint32_t*>(sv + 16));
        tmem_ld32(tDP + 32, reinterpret_cast<uint32_t*>(dp + 16));
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint32_t dk[16];
          if (j >= n_unmasked)
            ds_cols_by_key<BF16, true>(sv + 16 * g, dp + 16 * g, nm, c2, nl, nd, lim - 32 * g, dk);
          else
            ds_cols_by_key<BF16, false>(sv + 16 * g, dp + 16 * g, nm, c2, nl, nd, 32, dk);
          tmem_st16(tDP + 16 * g, dk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(B_DS + hk));
    }
    ok = mbar_wait_warp(bar(B_ACC), 0, ctl, 27) && ok;
    if (ok) {
      tc_fence_after();
      uint8_t* grow = reinterpret_cast<uint8_t*>(p.dq) +
                      2 * (b * p.dq_sb + h * p.dq_sh + static_cast<long long>(row) * p.dq_ss);
      store_acc_row<BF16>(tmem + Cfg::TM_ACC0 + lane_base, hk * (D / 2), D / 2, p.scale, grow, row < p.Sq);
    }
  }

#ifdef KFA_PROFILE
  prof_acc[0] = clock64() - prof_t0;
  if (lane == 0 && (warp == 0 || warp == 4 || warp == 8 || warp == 9))
    kfa_prof_flush(prof_acc, warp == 0 ? 0 : (warp == 4 ? 1 : (warp == 8 ? 2 : 3)));
#endif
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

}  // namespace kfa
