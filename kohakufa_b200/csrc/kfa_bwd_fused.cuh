// Attention backward for sm_100a as ONE key-major kernel: dK, dV and dQ from one P and one dS per
// (key tile, query tile) pair, five MMAs per pair
//     S^T = K Q_i^T     dP^T = V dO_i^T     dV += P^T dO_i     dQ_i = dS K     dK += dS^T Q_i
// as the reference's backward does (src/kohakufa/sm100/bwd.py:565-694 MMAs, 967-1127 P / dS
// partitions, 1135-1232 reduce partition), with two helper kernels around it:
//     kfa_bwd_prepare_kernel     (kfa_bwd.cuh) statistics, and here also zero-fills the dQ accumulator
//     kfa_bwd_dq_convert_kernel  dq = 16-bit(scale * accumulator)           (bwd.py:1391-1410)
//
// One CTA per (batch, K / V head, 128-key tile); it loops over the query tiles that see its keys (and
// over the query heads of its group). K and V stay in shared memory; Q_i and dO_i stream through rings.
// 512 threads, four warpgroups with register budgets of their own (setmaxnreg):
//   warps 0-3 / 4-7   P^T and dS^T for query columns 0-63 / 64-127 of every tile (thread <-> key row),
//                     then the dV / dK epilogue
//   warps 8-11        dQ: each finished dQ_i tile goes TMEM -> registers -> fp32 reduce-adds into the
//                     accumulator in global memory (thread <-> query row)
//   warp 12           MMA issue (converged, one elected lane issues)
//   warp 13 / 14      TMA producers: K, V, then the Q ring / the dO ring
// dS^T is written once, to shared memory (128-byte swizzled [key][query] boxes): the dK MMA reads it
// as a K-major A operand, the dQ MMA reads the same bytes as an MN-major (transposed) A operand
// (bwd.py:614-618). P^T goes to tensor memory over the S^T columns it came from (A operand of dV).
//
// Tensor memory (512 columns): S^T 128 | dP^T 128 | dV D | dK D | dQ D. At D = 128 that is 640, so dQ_i
// shares the dP^T columns (bwd.py:46-51): dQ(i) is issued once both warpgroups have read dP^T(i), and
// dP^T(i+1) once warps 8-11 hold dQ(i) in registers.
//
// The dQ accumulator is private scratch, so its layout is chosen for the adds: per (batch, head,
// 128-query tile) a block of 128 x D floats ordered [D / 4][128 rows][4], which makes every warp-wide
// red.global.add.v4.f32 cover 512 contiguous bytes (measured on B200: 6.4 TB/s of adds in that form,
// 3.5 TB/s with one row per lane in row-major order). Key tiles of one head start their walk over the
// query tiles at different places, so CTAs that run together add to different tiles (bwd.py:260-272).
// The order of the adds is not fixed: dQ is reproducible to rounding, not bit for bit (dK, dV are).
//
// Numerics: exactly those of the split kernels (kfa_bwd.cuh): P from the two separate statistics,
// unscaled 16-bit dS, scale applied to the fp32 dK and dQ, exact zeros for hidden / padded pairs.
#pragma once

#include "kfa_bwd.cuh"

namespace kfa {

constexpr int FUSED_THREADS = 512;
// Registers per thread: the kernel starts with 128 everywhere (512 threads x 128 = the whole register
// file); the dQ warpgroup and the MMA + TMA warpgroup then hand registers to the P / dS warpgroups:
// 2 x 128 x 144 + 128 x 152 + 128 x 72 = 65536 (the dQ warpgroup holds a whole 128 x 128 fp32 tile).
constexpr int FUSED_REGS_COMPUTE = 144, FUSED_REGS_REDUCE = 152, FUSED_REGS_ISSUE = 72;
static_assert(2 * 128 * FUSED_REGS_COMPUTE + 128 * FUSED_REGS_REDUCE + 128 * FUSED_REGS_ISSUE <= 512 * 128,
              "register budgets exceed the CTA's allocation (512 threads x 128): a setmaxnreg.inc would wait for ever");

template <int D>
struct FusedCfg {
  static constexpr int CHUNKS = D / 64;
  static constexpr int TILE_BYTES = CHUNKS * TILE_BYTES_64;
  // Q_i is read first by S^T(i) and last by dK(i), a whole step later, and S^T(i+1) is issued before
  // dK(i): three slots let the copy of Q_(i+2) start a step ahead. dO_i is done after dV(i), long
  // before dP^T(i+1) can be issued: one slot is enough at D = 128 (where no more fit), two at D = 64.
  static constexpr int NQ = 3;
  static constexpr int NDO = (D == 128) ? 1 : 2;
  static constexpr int DS_BYTES = 2 * TILE_BYTES_64;  // dS^T: two [128 keys][64 queries] boxes
  // How a finished dQ tile reaches the accumulator. D = 64: through two shared-memory staging buffers (128
  // rows x 32 columns fp32 each) and bulk reduce-adds by the copy engine. D = 128: no shared memory is left
  // for staging, the warpgroup issues the reduce-adds from registers (measured at D = 64: 10 % slower).
  static constexpr bool DQ_VIA_COPY_ENGINE = (D == 64);
  static constexpr int STAGE_BYTES = DQ_VIA_COPY_ENGINE ? 2 * 128 * 32 * 4 : 0;
  static constexpr int SMEM_TILES = (2 + NQ + NDO) * TILE_BYTES + DS_BYTES + STAGE_BYTES;
  // per-query statistics of a step: (-m, -log2 l) double-buffered (read by the P phase), -delta single
  // (read by the dS phase, reloaded while the next P phase runs)
  static constexpr int ML_BYTES = 2 * 128 * 4, DELTA_BYTES = 128 * 4;
  static constexpr int STATS_SMEM = 2 * ML_BYTES + DELTA_BYTES;
  // At D = 128 the tiles fill the 227 KB to within 3 KB: no room for alignment slack, the kernel relies on
  // (and checks) a 1024-byte aligned dynamic shared memory base.
  static constexpr int ALIGN_SLACK = (D == 128) ? 0 : 1024;
  static constexpr int SMEM_BYTES = SMEM_TILES + STATS_SMEM + 256 /*barriers*/ + ALIGN_SLACK;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + D;
  static constexpr uint32_t TM_DQ = (D == 128) ? TM_DP : 256 + 2 * D;
  static constexpr bool DQ_ALIASES_DP = (D == 128);
};
static_assert(FusedCfg<128>::SMEM_BYTES <= 232448 && FusedCfg<64>::SMEM_BYTES <= 232448, "shared memory");

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Instruction descriptor with the A operand MN-major as well (bit 15): dQ = dS K reads dS^T's shared-memory
// tile transposed.
__host__ __device__ constexpr uint32_t make_idesc_amn(bool bf16, int m, int n) {
  return make_idesc(bf16, true, m, n) | (1u << 15);
}

// dS^T = (dP^T - delta) * P of the same elements, rounded once to 16 bits, unscaled, written to the
// 128-byte swizzled [key][64 queries] box of this warpgroup: element order as above, so word
// (key row, query pair 8j + 2(lane % 4)) lands in 16-byte chunk j ^ (row % 8) of its row.
// nd: -delta of this thread's first column, in shared memory.
template <bool BF16>
__device__ __forceinline__ void ds_frag_to_smem(const float2* dp, const float2* pr, const float* nd_s, uint32_t s_row0,
                                                int lane) {
  const uint32_t sw = static_cast<uint32_t>(lane >> 2);  // row % 8 of every row this thread owns
  const uint32_t word = static_cast<uint32_t>(lane & 3) * 4u;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 nd = *reinterpret_cast<const float2*>(nd_s + 8 * j);
    const uint32_t col = ((static_cast<uint32_t>(j) ^ sw) << 4) + word;
#pragma unroll
    for (int e = 0; e < 4; ++e) {  // e = 2 * half + sel: row offset 16 * half + 8 * sel
      const int idx = 16 * (e >> 1) + 2 * j + (e & 1);
      const float2 d = __fmul2_rn(__fadd2_rn(dp[idx], nd), pr[idx]);
      const uint32_t w = pack16<BF16>(d.x, d.y);
      const uint32_t addr = s_row0 + static_cast<uint32_t>(16 * (e >> 1) + 8 * (e & 1)) * 128u + col;
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(w) : "memory");
    }
  }
}

// acc[128 x D] (+)= A[128 x 128] * B[128 rows, D]: A K-major in shared memory (two [128][64] boxes 16 KB
// apart), B MN-major (rows are the contraction index, boxes of 64 columns 16 KB apart).
template <int D>
__device__ __forceinline__ void issue_smemA_kmajor_bmn(bool lead, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                       uint32_t idesc, bool acc) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint32_t a_off = ((kk >> 2) * TILE_BYTES_64 + (kk & 3) * 32) >> 4;
    umma_ss_lead(lead, d_tmem, a_lo + a_off, b_lo + ((kk * 16 * 128) >> 4), idesc, (acc || kk > 0) ? 1u : 0u);
  }
}
// acc[128 x D] = A^T B: A stored [contraction][128] (MN-major, 64-column boxes 16 KB apart), B MN-major.
template <int D>
__device__ __forceinline__ void issue_smemA_mnmajor_bmn(bool lead, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                        uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint32_t off = (kk * 16 * 128) >> 4;
    umma_ss_lead(lead, d_tmem, a_lo + off, b_lo + off, idesc, kk > 0 ? 1u : 0u);
  }
}

// Floats of the dQ accumulator per (batch, head): whole 128-row tiles of D columns.
__host__ __device__ inline long long dq_acc_head_floats(int Sq, int D) {
  return static_cast<long long>((Sq + 127) / 128) * 128 * D;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(FUSED_THREADS, 1)
kfa_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const BwdParams p, float* __restrict__ dq_acc) {
  using Cfg = FusedCfg<D>;
  constexpr int CH = Cfg::CHUNKS;
  constexpr int NQ = Cfg::NQ, NDO = Cfg::NDO;
  constexpr int TB = Cfg::TILE_BYTES;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + static_cast<uint32_t>(Cfg::ALIGN_SLACK ? 1023 : 0)) & ~static_cast<uint32_t>(Cfg::ALIGN_SLACK ? 1023 : 0);
  if ((smem_base & 1023u) != 0u) {  // (never seen; the swizzled tiles would be garbage: report and leave)
    if (threadIdx.x == 0) atomicCAS(p.status, 0, KFA_DEV_BAD_SMEM_BASE);
    return;
  }
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sK = smem_base;
  const uint32_t sV = smem_base + TB;
  const uint32_t sQ = smem_base + 2 * TB;           // ring of NQ
  const uint32_t sDO = sQ + NQ * TB;                // ring of NDO
  const uint32_t sDS = sDO + NDO * TB;              // dS^T
  const uint32_t sStage = sDS + Cfg::DS_BYTES;       // dQ staging (if any)
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
  constexpr int B_DP = B_S + 1;                // dP^T(i) in TMEM
  constexpr int B_PLO = B_S + 2;               // the first 32 queries of P^T(i) stored by both warpgroups
  constexpr int B_P = B_S + 3;                 // P^T(i) stored by both warpgroups (256 arrivals)
  constexpr int B_DS = B_S + 4;                // dS^T(i) in shared memory, dP^T(i) read by both warpgroups
  constexpr int B_DSFREE = B_S + 5;            // dQ(i) and dK(i) have read dS^T(i)
  constexpr int B_DQ = B_S + 6;                // dQ(i) in TMEM
  constexpr int B_DQFREE = B_S + 7;            // dQ(i) copied to registers (128 arrivals)
  constexpr int B_ACC = B_S + 8;               // dV, dK complete
  constexpr int B_DRAIN = B_S + 9;
  constexpr int B_MLREADY = B_S + 10;          // 2   (-m, -log2 l) of a step landed
  constexpr int B_MLFREE = B_S + 12;           // 2   both warpgroups are done with them (256 arrivals)
  constexpr int B_DLREADY = B_S + 14;          // -delta of a step landed
  constexpr int B_DLFREE = B_S + 15;           // both warpgroups are done with it (256 arrivals)
  constexpr int B_STGFREE = B_S + 16;          // dQ staging: the buffer about to be written has been read out
  constexpr int B_STGFULL = B_S + 17;          // dQ staging: all 128 threads have written their part
  constexpr int N_BARS = B_S + 18;
  static_assert(N_BARS * 8 + 16 <= 256, "barrier block too small");
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // tile decode (groups of heads, tile-major inside); under a causal mask the first key tiles see the most queries and come first
  int bh, kt;  // bh over batch x K / V heads
  decode_tile(blockIdx.x, p.B * p.Hkv, p.n_k128, bh, kt);
  const int b = bh / p.Hkv, hk = bh % p.Hkv;
  const int kv0 = kt * 128;
  const int Sq = p.Sq, Skv = p.Skv;
  const int first_i = (p.P > 0) ? static_cast<int>((static_cast<long long>(kv0 / p.P) * p.P) / 128) : 0;
  const int n_per = max((Sq + 127) / 128 - first_i, 0);  // query tiles that see these keys
  const int n_steps = n_per * p.group;                   // ... for every query head of the group
  const bool ragged_keys = kv0 + 128 > Skv;
  const int i_full = (p.P > 0 && !ragged_keys) ? first_full_tile(kv0, p.P) : 0;  // query tiles before it are masked steps
  // step s -> query head, query tile. Key tile kt starts its walk kt tiles in, so that the CTAs of a head
  // that run side by side add their dQ tiles to different places.
  const int rot = (n_per > 0) ? kt % n_per : 0;
  auto tile_of = [&](int s) {
    int r = s % n_per + rot;
    if (r >= n_per) r -= n_per;
    return first_i + r;
  };
  auto head_of = [&](int s) { return hk * p.group + s / n_per; };
  auto tile_at = [&](const StepWalk& w) {  // the same without a division, for the loops that walk step by step
    int r = w.rel + rot;
    if (r >= n_per) r -= n_per;
    return first_i + r;
  };

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
    mbar_init(bar(B_DP), 1);
    mbar_init(bar(B_PLO), 256);
    mbar_init(bar(B_P), 256);
    mbar_init(bar(B_DS), 256);
    mbar_init(bar(B_DSFREE), 1);
    mbar_init(bar(B_DQ), 1);
    mbar_init(bar(B_DQFREE), 128);
    mbar_init(bar(B_ACC), 1);
    mbar_init(bar(B_DRAIN), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_MLREADY + i), 1);
      mbar_init(bar(B_MLFREE + i), 256);
    }
    mbar_init(bar(B_DLREADY), 1);
    mbar_init(bar(B_DLFREE), 256);
    mbar_init(bar(B_STGFREE), 1);
    mbar_init(bar(B_STGFULL), 128);
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

  // Each role sets its own register budget first thing: the issue warpgroup (warps 12-15) gives registers
  // up, the others wait until theirs are available.
  if (dead) {
  } else if (warp == 15) {
    // =========================== copies of the per-query statistics ===========================
    reg_budget<FUSED_REGS_ISSUE>();
    if (lane == 0 && n_steps > 0) {
      bool ok = true;
      int ml_issued = 0, dl_issued = 0;
      for (int s = 0; s < n_steps; ++s) {
        const float* src = p.stats + (static_cast<long long>(b) * p.H + head_of(s)) * p.stats_sh + tile_of(s) * 384ll;
        const int slot = s & 1, use = s >> 1;
        if (use > 0) ok = mbar_wait(bar(B_MLFREE + slot), (use - 1) & 1, ctl, 48);
        if (!ok) break;
        mbar_expect_tx(bar(B_MLREADY + slot), Cfg::ML_BYTES);
        bulk_load(sML + slot * Cfg::ML_BYTES, src, Cfg::ML_BYTES, bar(B_MLREADY + slot));
        ml_issued = s + 1;
        if (s > 0) ok = mbar_wait(bar(B_DLFREE), (s - 1) & 1, ctl, 49);
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
  } else if (warp == 13) {
    // =========================== TMA producer: K, V, then the Q ring ===========================
    reg_budget<FUSED_REGS_ISSUE>();
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
        if (use > 0) ok = mbar_wait(bar(B_QFREE + slot), (use - 1) & 1, ctl, 31);
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
  } else if (warp == 14) {
    // =========================== TMA producer: the dO ring ===========================
    reg_budget<FUSED_REGS_ISSUE>();
    if (lane == 0 && n_steps > 0) {
      prefetch_tensormap(&tmDO);
      bool ok = true;
      int issued = 0;
      for (int s = 0; s < n_steps; ++s) {
        const int slot = s % NDO, use = s / NDO;
        if (use > 0) ok = mbar_wait(bar(B_DOFREE + slot), (use - 1) & 1, ctl, 32);
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
  } else if (warp == 12) {
    // =========================== MMA issue ===========================
    reg_budget<FUSED_REGS_ISSUE>();
    if (n_steps > 0) {
      const bool lead = elect_one();
      constexpr uint32_t IDESC_S = make_idesc(BF16, false, 128, 128);   // A, B K-major
      constexpr uint32_t IDESC_ACC = make_idesc(BF16, true, 128, D);    // A K-major (or TMEM), B MN-major
      constexpr uint32_t IDESC_DQ = make_idesc_amn(BF16, 128, D);       // A, B MN-major
      const uint32_t tST = tmem + Cfg::TM_S, tDP = tmem + Cfg::TM_DP;
      const uint32_t tDV = tmem + Cfg::TM_DV, tDK = tmem + Cfg::TM_DK, tDQ = tmem + Cfg::TM_DQ;
      const uint32_t k_lo = sdesc_lo(sK, 16), v_lo = sdesc_lo(sV, 16);
      const uint32_t k_mn_lo = sdesc_lo(sK, TILE_BYTES_64);
      const uint32_t ds_k_lo = sdesc_lo(sDS, 16), ds_mn_lo = sdesc_lo(sDS, TILE_BYTES_64);
      bool ok = mbar_wait_warp(bar(B_KV), 0, ctl, 33);
      if (ok) ok = mbar_wait_warp(bar(B_QREADY + 0), 0, ctl, 34);
      if (ok) {
        tc_fence_after();
        issue_kmajor_n128<D>(lead, tST, k_lo, sdesc_lo(sQ, 16), IDESC_S);
        umma_commit_lead(lead, bar(B_S));
        ok = mbar_wait_warp(bar(B_DOREADY + 0), 0, ctl, 35);
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
        // dV += P^T(s) dO_s in two parts (the first 32 queries of each warpgroup's P^T are signalled
        // early), then S^T(s+1) may overwrite the P^T columns
        ok = mbar_wait_warp(bar(B_PLO), s & 1, ctl, 36);
        if (!ok) break;
        tc_fence_after();
        issue_tmemA_k64<D>(lead, tDV, tST, sdesc_lo(do_s, TILE_BYTES_64), IDESC_ACC, s > 0, 0);
        ok = mbar_wait_warp(bar(B_P), s & 1, ctl, 37);
        if (!ok) break;
        tc_fence_after();
        issue_tmemA_k64<D>(lead, tDV, tST, sdesc_lo(do_s, TILE_BYTES_64), IDESC_ACC, s > 0, 1);
        umma_commit_lead(lead, bar(B_DOFREE + s % NDO));
        if (more) {
          ok = mbar_wait_warp(bar(B_QREADY + (s + 1) % NQ), ((s + 1) / NQ) & 1, ctl, 38);
          if (!ok) break;
          tc_fence_after();
          issue_kmajor_n128<D>(lead, tST, k_lo, sdesc_lo(sQ + ((s + 1) % NQ) * TB, 16), IDESC_S);
          umma_commit_lead(lead, bar(B_S));
        }
        // dS^T(s) is in shared memory and dP^T(s) has been read: dQ_s = dS K (into columns of its own, or
        // over dP^T), dK += dS^T Q_s
        ok = mbar_wait_warp(bar(B_DS), s & 1, ctl, 39);
        if (!ok) break;
        if (!Cfg::DQ_ALIASES_DP && s > 0) {  // the previous dQ tile must have left its columns
          ok = mbar_wait_warp(bar(B_DQFREE), (s - 1) & 1, ctl, 40);
          if (!ok) break;
        }
        tc_fence_after();
        issue_smemA_mnmajor_bmn<D>(lead, tDQ, ds_mn_lo, k_mn_lo, IDESC_DQ);
        umma_commit_lead(lead, bar(B_DQ));
        issue_smemA_kmajor_bmn<D>(lead, tDK, ds_k_lo, sdesc_lo(q_s, TILE_BYTES_64), IDESC_ACC, s > 0);
        umma_commit_lead(lead, bar(B_QFREE + s % NQ));
        umma_commit_lead(lead, bar(B_DSFREE));
        if (more) {
          ok = mbar_wait_warp(bar(B_DOREADY + (s + 1) % NDO), ((s + 1) / NDO) & 1, ctl, 41);
          if (ok && Cfg::DQ_ALIASES_DP) ok = mbar_wait_warp(bar(B_DQFREE), s & 1, ctl, 42);
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
  } else if (warp >= 8 && warp < 12) {
    // =========================== dQ: TMEM -> registers -> reduce-adds ===========================
    reg_budget<FUSED_REGS_REDUCE>();
    const int r_in = tid & 127;
    const uint32_t tDQ = tmem + Cfg::TM_DQ + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    bool ok = true;
    StepWalk walk;
    for (int s = 0; s < n_steps; ++s, walk.next(n_per)) {
      const int i = tile_at(walk);
      const int head = hk * p.group + walk.g;
      ok = mbar_wait_warp(bar(B_DQ), s & 1, ctl, 43);
      if (!ok) break;
      tc_fence_after();
      // the whole tile goes to registers first, so that its columns are free at once (dP^T of the next step
      // is waiting for them at D = 128); the adds then drain at the rate the memory system takes them
      float v[D];
#pragma unroll
      for (int c = 0; c < D; c += 32) tmem_ld32(tDQ + c, reinterpret_cast<uint32_t*>(v + c));
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar(B_DQFREE));
      if constexpr (Cfg::DQ_VIA_COPY_ENGINE) {
        // Through shared memory to the copy engine: 32 columns (16 KB) at a time into one of two staging
        // buffers laid out like the accumulator ([4-column group][row][4]), each then added to global
        // memory by one bulk reduce. The thread that issues the copies (the warpgroup's first) also owns
        // their completion groups: before a buffer is rewritten, the reduce two commits back has read it.
        // The hand-shakes inside the warpgroup are bounded mbarrier waits, like every other wait here.
        float* tile = dq_acc + (static_cast<long long>(b) * p.H + head) * dq_acc_head_floats(Sq, D) +
                      static_cast<long long>(i) * (128 * D);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          const uint32_t buf = sStage + (c & 1) * 16384;
          const uint32_t n = static_cast<uint32_t>(s) * (D / 32) + c;  // running count of staged pieces
          if (tid == 256) {
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            mbar_arrive(bar(B_STGFREE));
          }
          ok = mbar_wait_warp(bar(B_STGFREE), n & 1, ctl, 29);
          if (!ok) break;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const uint32_t addr = buf + (g * 128 + r_in) * 16;
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[32 * c + 4 * g]),
                         "f"(v[32 * c + 4 * g + 1]), "f"(v[32 * c + 4 * g + 2]), "f"(v[32 * c + 4 * g + 3])
                         : "memory");
          }
          fence_async_smem();
          mbar_arrive(bar(B_STGFULL));
          if (tid == 256 && mbar_wait(bar(B_STGFULL), n & 1, ctl, 28)) {
            asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(tile + c * 4096),
                         "r"(buf), "r"(16384)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        if (!ok) break;
      } else {
        // Straight from registers; padded query rows hold exact zeros and are left out.
        float* dst = dq_acc + (static_cast<long long>(b) * p.H + head) * dq_acc_head_floats(Sq, D) +
                     static_cast<long long>(i) * (128 * D) + r_in * 4;
        if (i * 128 + r_in < Sq) {
#pragma unroll
          for (int c4 = 0; c4 < D / 4; ++c4)
            red_add_v4(dst + c4 * 512, v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
        }
      }
    }
    if (Cfg::DQ_VIA_COPY_ENGINE && tid == 256)
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // the staging buffers stay valid until read
  } else if (warp < 8) {
    // =========================== P^T / dS^T and the dV / dK epilogue ===========================
    reg_budget<FUSED_REGS_COMPUTE>();
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
    // dS^T box of this warpgroup, first row this thread writes
    const uint32_t s_row0 = sDS + hq * TILE_BYTES_64 + static_cast<uint32_t>((warp & 3) * 32 + (lane >> 2)) * 128u;
    const float2 c2 = make_float2(p.c, p.c);
    bool ok = true;
    StepWalk walk;
    for (int s = 0; s < n_steps; ++s, walk.next(n_per)) {
      const int i = tile_at(walk);
      const int q0 = i * 128 + 64 * hq + col0;  // query of this thread's first column
      // masked step: some (key, query) pair of this tile pair is hidden, or keys are padded
      const bool masked = ragged_keys || (p.P > 0 && i < i_full);
      const float* st = ml_smem + (s & 1) * (Cfg::ML_BYTES / 4) + 64 * hq + col0;  // -m here, -log2 l 128 floats on
      {  // both tests in flight together (the statistics have usually landed long before the scores)
        const bool ml_probe = mbar_test(bar(B_MLREADY + (s & 1)), (s >> 1) & 1);
        const bool s_probe = mbar_test(bar(B_S), s & 1);
        ok = mbar_wait_warp_probed(ml_probe, bar(B_MLREADY + (s & 1)), (s >> 1) & 1, ctl, 50);
        if (ok) ok = mbar_wait_warp_probed(s_probe, bar(B_S), s & 1, ctl, 44);
      }
      if (!ok) break;
      tc_fence_after();
      float2 pr[32];  // fp32 P of this thread's 64 elements, kept for the dS phase
      bool dp_probe, dsfree_probe, dl_probe;
      {
        float2 sv[32];
        tmem_ld_16x256b_x8(tS, reinterpret_cast<uint32_t*>(sv));
        tmem_ld_16x256b_x8(tS + HALF, reinterpret_cast<uint32_t*>(sv + 16));
        tmem_wait_ld();
        uint32_t pk[32];
        // 16-bit P^T goes over the first 32 of the 64 columns this warp has just read (all its lanes),
        // in two parts of 32 queries (16 packed columns) each
        if (masked)
          p_frag<BF16, true, 0>(sv, st, c2, q0, qmin, pr, pk);
        else
          p_frag<BF16, false, 0>(sv, st, c2, q0, qmin, pr, pk);
        tmem_st_16x128b_x4(tS, pk);
        tmem_st_16x128b_x4(tS + HALF, pk + 16);
        if constexpr (D == 128) {  // (at D = 64 the dV MMA is too short for the early start to pay)
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(bar(B_PLO));
        }
        // what the dS phase waits for is usually there by now: tested here, settled after the second half of P
        dp_probe = mbar_test(bar(B_DP), s & 1);
        dsfree_probe = (s == 0) || mbar_test(bar(B_DSFREE), (s - 1) & 1);
        dl_probe = mbar_test(bar(B_DLREADY), s & 1);
        if (masked)
          p_frag<BF16, true, 4>(sv, st, c2, q0, qmin, pr, pk);
        else
          p_frag<BF16, false, 4>(sv, st, c2, q0, qmin, pr, pk);
        tmem_st_16x128b_x4(tS + 16, pk + 8);
        tmem_st_16x128b_x4(tS + HALF + 16, pk + 24);
      }
      tmem_wait_st();
      tc_fence_before();
      if constexpr (D != 128) mbar_arrive(bar(B_PLO));
      mbar_arrive(bar(B_P));
      mbar_arrive(bar(B_MLFREE + (s & 1)));
      if (!__all_sync(0xffffffffu, dp_probe && dsfree_probe && dl_probe)) {
        ok = mbar_wait_warp(bar(B_DP), s & 1, ctl, 45);
        if (ok && s > 0) ok = mbar_wait_warp(bar(B_DSFREE), (s - 1) & 1, ctl, 46);
        if (ok) ok = mbar_wait_warp(bar(B_DLREADY), s & 1, ctl, 30);
      }
      if (!ok) break;
      tc_fence_after();
      {
        float2 dp[32];
        tmem_ld_16x256b_x8(tDP, reinterpret_cast<uint32_t*>(dp));
        tmem_ld_16x256b_x8(tDP + HALF, reinterpret_cast<uint32_t*>(dp + 16));
        tmem_wait_ld();
        ds_frag_to_smem<BF16>(dp, pr, dl_smem + 64 * hq + col0, s_row0, lane);
      }
      fence_async_smem();  // the MMAs read dS^T through the async proxy
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
      ok = mbar_wait_warp(bar(B_ACC), 0, ctl, 47) && ok;
      if (ok) {
        tc_fence_after();
        const uint32_t tacc = tmem + (hq ? Cfg::TM_DK : Cfg::TM_DV) + lane_base;
        store_acc_row<BF16>(tacc, 0, D, hq ? p.scale : 1.0f, grow, valid);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) {  // gave up (or an earlier kernel did): dK, dV rows of this CTA read as NaN (dQ: see the convert kernel)
    const int r1 = min(kv0 + 128, Skv);
    fill_rows_nan16(reinterpret_cast<uint8_t*>(p.dk) + 2 * (b * p.dk_sb + hk * p.dk_sh), p.dk_ss, kv0, r1, D);
    fill_rows_nan16(reinterpret_cast<uint8_t*>(p.dv) + 2 * (b * p.dv_sb + hk * p.dv_sh), p.dv_ss, kv0, r1, D);
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// dq = 16-bit(scale * accumulator), or NaN if the status word says that a kernel gave up: one CTA per (128-query tile, batch x head); the accumulator tile is
// [D / 4][128 rows][4] floats (see above), so a warp reads 512 contiguous bytes per load.
template <int D, bool BF16>
__global__ void __launch_bounds__(256) kfa_bwd_dq_convert_kernel(const float* __restrict__ dq_acc, void* dq,
                                                                 long long dq_sb, long long dq_sh, long long dq_ss,
                                                                 int H, int Sq, float scale, const int* status) {
  const int tile = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh % H;
  const int r_in = threadIdx.x & 127, half = threadIdx.x >> 7;
  const int row = tile * 128 + r_in;
  if (row >= Sq) return;
  const float* src = dq_acc + static_cast<long long>(bh) * dq_acc_head_floats(Sq, D) +
                     static_cast<long long>(tile) * (128 * D) + r_in * 4;
  uint8_t* drow = reinterpret_cast<uint8_t*>(dq) + 2 * (b * dq_sb + h * dq_sh + static_cast<long long>(row) * dq_ss);
  if (*status != 0) {  // a kernel before this one gave up: the accumulator is incomplete
    for (int c8 = half * (D / 16); c8 < (half + 1) * (D / 16); ++c8)
      *reinterpret_cast<uint4*>(drow + 16 * c8) = make_uint4(0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu);
    return;
  }
#pragma unroll
  for (int c8 = half * (D / 16); c8 < (half + 1) * (D / 16); ++c8) {
    const float4 a = *reinterpret_cast<const float4*>(src + (2 * c8) * 512);
    const float4 c = *reinterpret_cast<const float4*>(src + (2 * c8 + 1) * 512);
    uint4 w;
    w.x = pack16<BF16>(a.x * scale, a.y * scale);
    w.y = pack16<BF16>(a.z * scale, a.w * scale);
    w.z = pack16<BF16>(c.x * scale, c.y * scale);
    w.w = pack16<BF16>(c.z * scale, c.w * scale);
    *reinterpret_cast<uint4*>(drow + 16 * c8) = w;
  }
}

}  // namespace kfa
