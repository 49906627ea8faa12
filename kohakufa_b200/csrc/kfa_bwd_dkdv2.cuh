// dK / dV kernel of the split backward, second form: P^T goes to shared memory instead of over the S^T
// columns of tensor memory, so that the next step's S^T = K Q^T can be issued as soon as the warpgroups
// hold the current scores in registers, instead of after dV has consumed P^T (with tensor memory full at
// D = 128 — S^T, dP^T, dV, dK: 4 x 128 columns — that dependence made every step a chain
// P -> dV -> next S^T -> next P; see kfa_bwd.cuh for the first form, which masks, packed batches and the
// context-parallel steps still use).
//
//   one CTA per (batch, K / V head, 128-key tile), looping over the query tiles that see it (and the
//   query heads of its group); keys on TMEM lanes:
//     S^T = K Q_i^T          both operands in shared memory, issued one step ahead
//     dP^T = V dO_i^T        both operands in shared memory
//     dV += P^T dO_i         A = P^T in shared memory (128-byte swizzled [key][query]), B = dO_i MN-major
//     dK += dS^T Q_i         A = dS^T in tensor memory over the dP^T columns, B = Q_i MN-major
//   (reference: src/kohakufa/sm100/bwd.py:565-694 MMAs, 967-1127 P / dS partitions)
//
// 384 threads: warps 0-3 / 4-7 compute P^T and dS^T for query columns 0-63 / 64-127 of every tile
// (4 keys x 16 queries per thread per phase, fragment-shaped TMEM access), warp 8 issues the MMAs,
// warps 9-11 are the copy producers (K, V and the Q ring; the dO ring; the per-step statistics).
// Shared memory at D = 128: K, V 64 KB, Q ring 3 x 32 KB, dO 1 x 32 KB, P^T 32 KB, statistics 2.5 KB:
// 226.75 KB, so the kernel relies on (and checks) a 1 KB aligned dynamic shared memory base.
// Numerics: exactly those of the first form (same operands, same accumulation order): bit-identical dK, dV.
#pragma once

#include "kfa_bwd_fused.cuh"

namespace kfa {

constexpr int DKDV2_THREADS = 384;

template <int D>
struct Dkdv2Cfg {
  static constexpr int CHUNKS = D / 64;
  static constexpr int TILE_BYTES = CHUNKS * TILE_BYTES_64;
  static constexpr int NQ = 3;                         // Q_i: read by S^T(i) a step early and by dK(i) last
  static constexpr int NDO = (D == 128) ? 1 : 2;       // dO_i: read by dP^T(i), then by dV(i)
  static constexpr int P_BYTES = 2 * TILE_BYTES_64;    // P^T: two [128 keys][64 queries] boxes
  static constexpr int SMEM_TILES = (2 + NQ + NDO) * TILE_BYTES + P_BYTES;
  static constexpr int ML_BYTES = 2 * 128 * 4, DELTA_BYTES = 128 * 4;
  static constexpr int STATS_SMEM = 2 * ML_BYTES + DELTA_BYTES;
  static constexpr int ALIGN_SLACK = (D == 128) ? 0 : 1024;
  static constexpr int SMEM_BYTES = SMEM_TILES + STATS_SMEM + 256 /*barriers*/ + ALIGN_SLACK;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + D;
};
static_assert(Dkdv2Cfg<128>::SMEM_BYTES <= 232448 && Dkdv2Cfg<64>::SMEM_BYTES <= 232448, "shared memory");

// The 16-bit P^T of the thread's 4 keys x 16 queries (element order of p_frag) into the 128-byte swizzled
// [key][64 queries] box of its warpgroup: word (key row, query pair 8j + 2(lane % 4)) lands in 16-byte
// chunk j ^ (row % 8) of its row.
__device__ __forceinline__ void p_words_to_smem(const uint32_t* pk, uint32_t s_row0, int lane) {
  const uint32_t sw = static_cast<uint32_t>(lane >> 2);
  const uint32_t word = static_cast<uint32_t>(lane & 3) * 4u;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t col = ((static_cast<uint32_t>(j) ^ sw) << 4) + word;
#pragma unroll
    for (int e = 0; e < 4; ++e) {  // e = 2 * half + sel: row offset 16 * half + 8 * sel
      const uint32_t addr = s_row0 + static_cast<uint32_t>(16 * (e >> 1) + 8 * (e & 1)) * 128u + col;
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(pk[16 * (e >> 1) + 2 * j + (e & 1)]) : "memory");
    }
  }
}

template <int D, bool BF16>
__global__ void __launch_bounds__(DKDV2_THREADS, 1)
kfa_bwd_dkdv2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const BwdParams p) {
  using Cfg = Dkdv2Cfg<D>;
  constexpr int CH = Cfg::CHUNKS;
  constexpr int NQ = Cfg::NQ, NDO = Cfg::NDO;
  constexpr int TB = Cfg::TILE_BYTES;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t ALIGN_MASK = Cfg::ALIGN_SLACK ? 1023u : 0u;
  const uint32_t smem_base = (smem_u32(smem_raw) + ALIGN_MASK) & ~ALIGN_MASK;
  if ((smem_base & 1023u) != 0u) {  // (never seen; the swizzled tiles would be garbage: report and leave)
    if (threadIdx.x == 0) atomicCAS(p.status, 0, KFA_DEV_BAD_SMEM_BASE);
    return;
  }
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sK = smem_base;
  const uint32_t sV = smem_base + TB;
  const uint32_t sQ = smem_base + 2 * TB;   // ring of NQ
  const uint32_t sDO = sQ + NQ * TB;        // ring of NDO
  const uint32_t sP = sDO + NDO * TB;       // P^T
  const uint32_t sML = smem_base + Cfg::SMEM_TILES;  // 2 x (-m[128], -log2 l[128])
  const uint32_t sDL = sML + 2 * Cfg::ML_BYTES;      // -delta[128]
  const float* ml_smem = reinterpret_cast<const float*>(smem + Cfg::SMEM_TILES);
  const float* dl_smem = ml_smem + 2 * Cfg::ML_BYTES / 4;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::SMEM_TILES + Cfg::STATS_SMEM);
  constexpr int B_KV = 0;                      // K, V landed
  constexpr int B_QREADY = 1;                  // NQ
  constexpr int B_QFREE = B_QREADY + NQ;       // NQ   dK(i), the last reader of Q_i, has retired
  constexpr int B_DOREADY = B_QFREE + NQ;      // NDO
  constexpr int B_DOFREE = B_DOREADY + NDO;    // NDO  dV(i), the last reader of dO_i, has retired
  constexpr int B_S = B_DOFREE + NDO;          // S^T(i) in TMEM
  constexpr int B_SREAD = B_S + 1;             // both warpgroups hold S^T(i) in registers (256 arrivals)
  constexpr int B_DP = B_S + 2;                // dP^T(i) in TMEM
  constexpr int B_P = B_S + 3;                 // P^T(i) in shared memory (256 arrivals)
  constexpr int B_PFREE = B_S + 4;             // dV(i) has read P^T(i)
  constexpr int B_DS = B_S + 5;                // dS^T(i) in TMEM (256 arrivals)
  constexpr int B_ACC = B_S + 6;               // dV, dK complete
  constexpr int B_DRAIN = B_S + 7;
  constexpr int B_MLREADY = B_S + 8;           // 2   (-m, -log2 l) of a step landed
  constexpr int B_MLFREE = B_S + 10;           // 2   both warpgroups are done with them (256 arrivals)
  constexpr int B_DLREADY = B_S + 12;          // -delta of a step landed
  constexpr int B_DLFREE = B_S + 13;           // both warpgroups are done with it (256 arrivals)
  constexpr int N_BARS = B_S + 14;
  static_assert(N_BARS * 8 + 16 <= 256, "barrier block too small");
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // tile decode: head-major; under a causal mask the first key tiles see the most queries and come first
  const int bh = blockIdx.x / p.n_k128;  // over batch x K / V heads
  const int kt = blockIdx.x % p.n_k128;
  const int b = bh / p.Hkv, hk = bh % p.Hkv;
  const int kv0 = kt * 128;
  const int Sq = p.Sq, Skv = p.Skv;
  const int first_i = (p.P > 0) ? static_cast<int>((static_cast<long long>(kv0 / p.P) * p.P) / 128) : 0;
  const int n_per = max((Sq + 127) / 128 - first_i, 0);  // query tiles that see these keys
  const int n_steps = n_per * p.group;                   // ... for every query head of the group
  const bool ragged_keys = kv0 + 128 > Skv;
  auto tile_of = [&](int s) { return first_i + s % n_per; };
  auto head_of = [&](int s) { return hk * p.group + s / n_per; };

  if (tid == 0) {
    mbar_init(bar(B_KV), 1);
    for (int i = 0; i < NQ; ++i) {
      mbar_init(bar(B_QREADY + i), 1);
      mbar_init(bar(B_QFREE + i), 1);
    }
    for (int i = 0; i < NDO; ++i) {
      mbar_init(bar(B_DOREADY + i), 1);
      mbar_init(bar(B_DOFREE + i), 1);
    }
    mbar_init(bar(B_S), 1);
    mbar_init(bar(B_SREAD), 256);
    mbar_init(bar(B_DP), 1);
    mbar_init(bar(B_P), 256);
    mbar_init(bar(B_PFREE), 1);
    mbar_init(bar(B_DS), 256);
    mbar_init(bar(B_ACC), 1);
    mbar_init(bar(B_DRAIN), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_MLREADY + i), 1);
      mbar_init(bar(B_MLFREE + i), 256);
    }
    mbar_init(bar(B_DLREADY), 1);
    mbar_init(bar(B_DLFREE), 256);
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
  const Ctl ctl{s_abort, p.status};
  const bool dead = (*s_abort != 0);

  if (dead) {
  } else if (warp == 9) {
    // =========================== copies: K, V, then the Q ring ===========================
    if (lane == 0 && n_steps > 0) {
      prefetch_tensormap(&tmQ);
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmV);
      mbar_expect_tx(bar(B_KV), 2 * TB);
      for (int ch = 0; ch < CH; ++ch) {
        tma_load_4d(sK + ch * TILE_BYTES_64, &tmK, bar(B_KV), ch * 64, kv0, hk, b);
        tma_load_4d(sV + ch * TILE_BYTES_64, &tmV, bar(B_KV), ch * 64, kv0, hk, b);
      }
      bool ok = true;
      int issued = 0;
      for (int s = 0; s < n_steps; ++s) {
        const int slot = s % NQ, use = s / NQ;
        if (use > 0) ok = mbar_wait(bar(B_QFREE + slot), (use - 1) & 1, ctl, 71);
        if (!ok) break;
        mbar_expect_tx(bar(B_QREADY + slot), TB);
        for (int ch = 0; ch < CH; ++ch)
          tma_load_4d(sQ + slot * TB + ch * TILE_BYTES_64, &tmQ, bar(B_QREADY + slot), ch * 64, tile_of(s) * 128,
                      head_of(s), b);
        issued = s + 1;
      }
      if (!ok) {  // aborting: let the copies in flight land before the CTA gives up its shared memory
        mbar_drain(bar(B_KV), 0);
        for (int s = max(issued - NQ, 0); s < issued; ++s) mbar_drain(bar(B_QREADY + s % NQ), (s / NQ) & 1);
      }
    }
  } else if (warp == 10) {
    // =========================== copies: the dO ring ===========================
    if (lane == 0 && n_steps > 0) {
      prefetch_tensormap(&tmDO);
      bool ok = true;
      int issued = 0;
      for (int s = 0; s < n_steps; ++s) {
        const int slot = s % NDO, use = s / NDO;
        if (use > 0) ok = mbar_wait(bar(B_DOFREE + slot), (use - 1) & 1, ctl, 72);
        if (!ok) break;
        mbar_expect_tx(bar(B_DOREADY + slot), TB);
        for (int ch = 0; ch < CH; ++ch)
          tma_load_4d(sDO + slot * TB + ch * TILE_BYTES_64, &tmDO, bar(B_DOREADY + slot), ch * 64, tile_of(s) * 128,
                      head_of(s), b);
        issued = s + 1;
      }
      if (!ok)
        for (int s = max(issued - NDO, 0); s < issued; ++s) mbar_drain(bar(B_DOREADY + s % NDO), (s / NDO) & 1);
    }
  } else if (warp == 11) {
    // =========================== copies: the per-query statistics ===========================
    if (lane == 0 && n_steps > 0) {
      bool ok = true;
      int ml_issued = 0, dl_issued = 0;
      for (int s = 0; s < n_steps; ++s) {
        const float* src = p.stats + (static_cast<long long>(b) * p.H + head_of(s)) * p.stats_sh + tile_of(s) * 384ll;
        const int slot = s & 1, use = s >> 1;
        if (use > 0) ok = mbar_wait(bar(B_MLFREE + slot), (use - 1) & 1, ctl, 73);
        if (!ok) break;
        mbar_expect_tx(bar(B_MLREADY + slot), Cfg::ML_BYTES);
        bulk_load(sML + slot * Cfg::ML_BYTES, src, Cfg::ML_BYTES, bar(B_MLREADY + slot));
        ml_issued = s + 1;
        if (s > 0) ok = mbar_wait(bar(B_DLFREE), (s - 1) & 1, ctl, 74);
        if (!ok) break;
        mbar_expect_tx(bar(B_DLREADY), Cfg::DELTA_BYTES);
        bulk_load(sDL, src + 256, Cfg::DELTA_BYTES, bar(B_DLREADY));
        dl_issued = s + 1;
      }
      if (!ok) {
        for (int s = max(ml_issued - 2, 0); s < ml_issued; ++s) mbar_drain(bar(B_MLREADY + (s & 1)), (s >> 1) & 1);
        if (dl_issued > 0) mbar_drain(bar(B_DLREADY), (dl_issued - 1) & 1);
      }
    }
  } else if (warp == 8) {
    // =========================== MMA issue ===========================
    if (n_steps > 0) {
      const bool lead = elect_one();
      constexpr uint32_t IDESC_S = make_idesc(BF16, false, 128, 128);   // A, B K-major
      constexpr uint32_t IDESC_ACC = make_idesc(BF16, true, 128, D);    // A K-major (or TMEM), B MN-major
      const uint32_t tST = tmem + Cfg::TM_S, tDP = tmem + Cfg::TM_DP;
      const uint32_t tDV = tmem + Cfg::TM_DV, tDK = tmem + Cfg::TM_DK;
      const uint32_t k_lo = sdesc_lo(sK, 16), v_lo = sdesc_lo(sV, 16);
      const uint32_t p_lo = sdesc_lo(sP, 16);
      bool ok = mbar_wait_warp(bar(B_KV), 0, ctl, 75);
      if (ok) ok = mbar_wait_warp(bar(B_QREADY + 0), 0, ctl, 76);
      if (ok) {
        tc_fence_after();
        issue_kmajor_n128<D>(lead, tST, k_lo, sdesc_lo(sQ, 16), IDESC_S);
        umma_commit_lead(lead, bar(B_S));
        ok = mbar_wait_warp(bar(B_DOREADY + 0), 0, ctl, 77);
      }
      if (ok) {
        tc_fence_after();
        issue_kmajor_n128<D>(lead, tDP, v_lo, sdesc_lo(sDO, 16), IDESC_S);
        umma_commit_lead(lead, bar(B_DP));
      }
      for (int s = 0; s < n_steps && ok; ++s) {
        const uint32_t q_s = sQ + (s % NQ) * TB;
        const uint32_t do_s = sDO + (s % NDO) * TB;
        const bool more = s + 1 < n_steps;
        if (more) {  // S^T(s+1), as soon as the warpgroups hold S^T(s) in registers
          ok = mbar_wait_warp(bar(B_QREADY + (s + 1) % NQ), ((s + 1) / NQ) & 1, ctl, 78);
          if (ok) ok = mbar_wait_warp(bar(B_SREAD), s & 1, ctl, 79);
          if (!ok) break;
          tc_fence_after();
          issue_kmajor_n128<D>(lead, tST, k_lo, sdesc_lo(sQ + ((s + 1) % NQ) * TB, 16), IDESC_S);
          umma_commit_lead(lead, bar(B_S));
        }
        // dV += P^T(s) dO_s (P^T from shared memory)
        ok = mbar_wait_warp(bar(B_P), s & 1, ctl, 80);
        if (!ok) break;
        tc_fence_after();
        issue_smemA_kmajor_bmn<D>(lead, tDV, p_lo, sdesc_lo(do_s, TILE_BYTES_64), IDESC_ACC, s > 0);
        umma_commit_lead(lead, bar(B_PFREE));
        umma_commit_lead(lead, bar(B_DOFREE + s % NDO));
        // dK += dS^T(s) Q_s (dS^T in TMEM over the dP^T columns), then dP^T(s+1) may overwrite them
        ok = mbar_wait_warp(bar(B_DS), s & 1, ctl, 81);
        if (!ok) break;
        tc_fence_after();
        issue_tmemA_k128<D>(lead, tDK, tDP, sdesc_lo(q_s, TILE_BYTES_64), IDESC_ACC, s > 0);
        umma_commit_lead(lead, bar(B_QFREE + s % NQ));
        if (more) {
          ok = mbar_wait_warp(bar(B_DOREADY + (s + 1) % NDO), ((s + 1) / NDO) & 1, ctl, 82);
          if (!ok) break;
          tc_fence_after();
          issue_kmajor_n128<D>(lead, tDP, v_lo, sdesc_lo(sDO + ((s + 1) % NDO) * TB, 16), IDESC_S);
          umma_commit_lead(lead, bar(B_DP));
        }
      }
      if (ok) umma_commit_lead(lead, bar(B_ACC));
      umma_commit_lead(lead, bar(B_DRAIN));
      mbar_drain(bar(B_DRAIN), 0);
    }
  } else if (warp < 8) {
    // =========================== P^T / dS^T and the dV / dK epilogue ===========================
    const int hq = warp >> 2;  // which 64 query columns of every tile
    const int k_in = tid & 127;
    const int key = kv0 + k_in;  // the epilogue's row (one TMEM lane per thread)
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + Cfg::TM_S + 64 * hq + lane_base;
    const uint32_t tDP = tmem + Cfg::TM_DP + 64 * hq + lane_base;
    constexpr uint32_t HALF = 16u << 16;  // the warp's second 16 lanes
    // In the compute phases a thread works on 4 key rows x 16 query columns (see p_frag):
    // first query that sees each of its keys; padded keys see nothing
    const int col0 = 2 * (lane & 3);  // its first column inside every block of 8
    int qmin[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kr = kv0 + (warp & 3) * 32 + 16 * (e >> 1) + (lane >> 2) + 8 * (e & 1);
      qmin[e] = 0;
      if (kr >= Skv) qmin[e] = 0x7fffffff;
      else if (p.P > 0) qmin[e] = (kr / p.P) * p.P;
    }
    // P^T box of this warpgroup, first row this thread writes
    const uint32_t s_row0 = sP + hq * TILE_BYTES_64 + static_cast<uint32_t>((warp & 3) * 32 + (lane >> 2)) * 128u;
    const float2 c2 = make_float2(p.c, p.c);
    bool ok = true;
    for (int s = 0; s < n_steps; ++s) {
      const int i = tile_of(s);
      const int q0 = i * 128 + 64 * hq + col0;  // query of this thread's first column
      // masked step: some (key, query) pair of this tile pair is hidden, or keys are padded
      const bool masked = ragged_keys || (p.P > 0 && key_limit(i * 128, p.P, Skv) < kv0 + 128);
      const float* st = ml_smem + (s & 1) * (Cfg::ML_BYTES / 4) + 64 * hq + col0;  // -m here, -log2 l 128 floats on
      ok = mbar_wait_warp(bar(B_MLREADY + (s & 1)), (s >> 1) & 1, ctl, 83);
      if (ok) ok = mbar_wait_warp(bar(B_S), s & 1, ctl, 84);
      if (!ok) break;
      tc_fence_after();
      float2 pr[32];  // fp32 P of this thread's 64 elements, kept for the dS phase
      {
        float2 sv[32];
        tmem_ld_16x256b_x8(tS, reinterpret_cast<uint32_t*>(sv));
        tmem_ld_16x256b_x8(tS + HALF, reinterpret_cast<uint32_t*>(sv + 16));
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(bar(B_SREAD));  // S^T(s) is in registers: the tensor core may write S^T(s+1)
        uint32_t pk[32];
        if (masked) {
          p_frag<BF16, true, 0>(sv, st, c2, q0, qmin, pr, pk);
          p_frag<BF16, true, 4>(sv, st, c2, q0, qmin, pr, pk);
        } else {
          p_frag<BF16, false, 0>(sv, st, c2, q0, qmin, pr, pk);
          p_frag<BF16, false, 4>(sv, st, c2, q0, qmin, pr, pk);
        }
        mbar_arrive(bar(B_MLFREE + (s & 1)));
        if (s > 0) ok = mbar_wait_warp(bar(B_PFREE), (s - 1) & 1, ctl, 85);  // dV(s-1) has read the buffer
        if (!ok) break;
        p_words_to_smem(pk, s_row0, lane);
      }
      fence_async_smem();  // the dV MMA reads P^T through the async proxy
      mbar_arrive(bar(B_P));
      ok = mbar_wait_warp(bar(B_DP), s & 1, ctl, 86);
      if (ok) ok = mbar_wait_warp(bar(B_DLREADY), s & 1, ctl, 87);
      if (!ok) break;
      tc_fence_after();
      {
        float2 dp[32];
        tmem_ld_16x256b_x8(tDP, reinterpret_cast<uint32_t*>(dp));
        tmem_ld_16x256b_x8(tDP + HALF, reinterpret_cast<uint32_t*>(dp + 16));
        tmem_wait_ld();
        uint32_t dk[32];
        ds_frag<BF16>(dp, pr, dl_smem - 256 + 64 * hq + col0, dk);  // (ds_frag reads -delta at its pointer + 256)
        tmem_st_16x128b_x8(tDP, dk);
        tmem_st_16x128b_x8(tDP + HALF, dk + 16);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(B_DS));
      mbar_arrive(bar(B_DLFREE));
    }
    // ---- epilogue: warps 0-3 store dV, warps 4-7 store scale * dK ----
    const bool valid = key < Skv;
    uint8_t* grow;
    if (hq == 0)
      grow = reinterpret_cast<uint8_t*>(p.dv) + 2 * (b * p.dv_sb + hk * p.dv_sh + static_cast<long long>(key) * p.dv_ss);
    else
      grow = reinterpret_cast<uint8_t*>(p.dk) + 2 * (b * p.dk_sb + hk * p.dk_sh + static_cast<long long>(key) * p.dk_ss);
    if (n_steps == 0) {
      if (valid)
        for (int cc = 0; cc < D; cc += 8) *reinterpret_cast<uint4*>(grow + 2 * cc) = make_uint4(0, 0, 0, 0);
    } else {
      ok = mbar_wait_warp(bar(B_ACC), 0, ctl, 88) && ok;
      if (ok) {
        tc_fence_after();
        const uint32_t tacc = tmem + (hq ? Cfg::TM_DK : Cfg::TM_DV) + lane_base;
        store_acc_row<BF16>(tacc, 0, D, hq ? p.scale : 1.0f, grow, valid);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) {  // gave up (or an earlier kernel did): the rows of this CTA read as NaN
    const int r1 = min(kv0 + 128, Skv);
    fill_rows_nan16(reinterpret_cast<uint8_t*>(p.dk) + 2 * (b * p.dk_sb + hk * p.dk_sh), p.dk_ss, kv0, r1, D);
    fill_rows_nan16(reinterpret_cast<uint8_t*>(p.dv) + 2 * (b * p.dv_sb + hk * p.dv_sh), p.dv_ss, kv0, r1, D);
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

}  // namespace kfa
