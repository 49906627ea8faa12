// Attention forward for sm_100a: O = softmax(scale * Q K^T + mask) V, plus the two per-row
// statistics m (row max of the raw, unscaled scores) and log2(l), l = sum exp2((S - m) * c),
// c = scale * log2(e).
//
// Replaces the reference's Gluon forward (src/kohakufa/sm100/fwd.py:1065-1136 kernel,
// 578-1039 partitions, 76-418 tile scheduler) with a hand-written kernel:
//
//   CTA = 256 query rows of one (batch, head), as two 128-row halves; key tiles of 128. 512 threads:
//   warps 0-3   softmax of half 0 (thread t <-> query row t): row max, exponentials, P, row sum
//   warps 4-7   the same for half 1
//   warps 8-11  correction for both halves: exact rescale of O_h whenever a row's max moved; runs beside
//               the exponentials
//   (epilogue: each softmax warpgroup writes its own half, O / l -> 16 bits -> global, statistics)
//   warps 12, 14  MMA issue for half 0 / half 1 (one lane each): S_h = Q_h K_j^T, O_h += P_h V_j  (tcgen05, TMEM)
//   warp  13    TMA producer (one lane): Q halves once, K_j / V_j through a ring
//   Register budgets per role (setmaxnreg): the softmax warpgroups take what the others give up.
//
//   TMEM columns: S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [256+D,256+2D).
//   A key tile's 128 score columns are produced and consumed as two parts of 64 keys: S_h part p sits in
//   columns 64p..64p+63 of S_h, its P (16-bit) overwrites the first 32 of them and is the A operand of
//   O_h += P V for those 64 keys. As soon as that MMA is issued the next tile's scores of the same part
//   follow into the same columns, while the softmax warpgroup works on the other part: neither waits for
//   a whole tile of the other. (The 64-column score MMAs run at 2/3 of the tensor core's rate, because both
//   operands stream from shared memory; the key loop was bound by the hand-offs, not by the tensor core.)
//
// Numerics kept from the reference (docs/precision.md:17-114; fwd.py:785-790, 905-924, 1029-1038):
//   * the exponent is shift-then-scale, exp2((S - m) * c): the row's largest P is exactly 1;
//   * m is the running max of the raw scores, with an exact rescale of O whenever it moves;
//   * l sums the unrounded fp32 P; m and log2(l) are stored as two separate fp32 numbers.
// Hidden key tiles of a causal / block-causal problem are never loaded: the key loop of a
// half stops at its last visible tile (fwd.py:243, 265).
#pragma once

#include "kfa_ptx.cuh"

namespace kfa {

struct FwdParams {
  void* o;  // [B, H, Sq, D] view; element strides; last dim contiguous
  long long o_sb, o_sh, o_ss;
  float* lse;  // [B, H, 2, Sq]: plane 0 = m, plane 1 = log2(l)
  int B, H, Sq, Skv;
  int P;    // 0 dense; P > 0: key c visible to query r iff c / P <= r / P
  float c;  // scale * log2(e)
  int n_q_tiles;
  int* status;
  int group;  // query heads per K / V head (grouped-query attention): K / V head of query head h is h / group
  // Context-parallel steps (mode != 0): instead of the normalised 16-bit O and (m, log2 l), the
  // kernel leaves the unnormalised fp32 O and (m, l) in a carry that the next step merges with.
  int mode;            // 0 normal; 1 write the carry; 2 merge with the existing carry and write it
  float* o_acc;        // fp32 rows of D, row r of (b, h) at o_acc + (b * H + h) * oa_sh + r * D
  long long oa_sh;
  float* ml;           // m at ml[(b * H + h) * ml_sh + r], l at the same + ml_plane
  long long ml_sh, ml_plane;
  // Packed variable-length batches (cu_q != nullptr): the tensors are [1, H, T, D]; sequence b (of B)
  // owns query rows cu_q[b] .. cu_q[b + 1] and key rows cu_k[b] .. cu_k[b + 1] and is its own attention
  // problem. Sq is then the tensors' row count T (it sizes the statistics planes) and n_q_tiles counts
  // the tiles of the longest sequence; CTAs past the end of a shorter one return at once.
  const int* cu_q;
  const int* cu_k;
  // Boolean mask (kernels instantiated with MASKW): 32 keys per word, bit set = visible; the words of
  // query row r of (b, h) start at mw + b * mw_sb + h * mw_sh + r * mw_row (a stride of 0 broadcasts),
  // four words per 128-key tile, zero bits for keys past Skv.
  const int* mw;
  long long mw_sb, mw_sh;
  int mw_row;
  // Optional with a mask: one int per (128 queries x 128 keys) tile, nonzero = some bit of the tile is set;
  // tile (qt, kt) of (b, h) at mt + b * mt_sb + h * mt_sh + qt * mt_row + kt. Key tiles in which neither
  // half of the CTA sees anything are skipped by every role (nullptr: all key tiles are visited).
  const int* mt;
  long long mt_sb, mt_sh;
  int mt_row;
};

// Longest list of visited tiles a CTA keeps in shared memory (masks with more tiles per row visit all).
constexpr int TILE_LIST_CAP = 1024;

constexpr int FWD_THREADS = 512;
// Registers per thread once the roles have set their budgets (the kernel starts with 128 each):
// 2 softmax warpgroups, the correction warpgroup, the MMA + TMA warpgroup: 2 x 128 x 152 + 128 x 96 + 128 x 96 = 63488 (one 128-key part per tile: 176 / 72 / 88).
#if defined(KFA_FWD_PARTS) && KFA_FWD_PARTS == 1
constexpr int FWD_REGS_SOFTMAX = 176, FWD_REGS_CORRECTION = 72, FWD_REGS_ISSUE = 88;
#else
constexpr int FWD_REGS_SOFTMAX = 152, FWD_REGS_CORRECTION = 96, FWD_REGS_ISSUE = 96;
#endif
// (A CTA owns the registers it was launched with, 512 x 128 here: budgets beyond that would make a
// setmaxnreg.inc wait for ever.)
static_assert(2 * 128 * FWD_REGS_SOFTMAX + 128 * FWD_REGS_CORRECTION + 128 * FWD_REGS_ISSUE <= FWD_THREADS * 128,
              "register budgets exceed the CTA's allocation");
#ifndef KFA_FWD_PARTS
#define KFA_FWD_PARTS 2
#endif
constexpr int FWD_PARTS = KFA_FWD_PARTS;       // pieces a key tile's 128 score columns are produced and consumed in
constexpr int FWD_PART_KEYS = 128 / FWD_PARTS;
constexpr int FWD_BAR_BYTES = 512;        // mbarriers + the tensor-memory address
constexpr int FWD_HANDOVER_BYTES = 2048;  // alpha [half][part][128], fp32
constexpr int TILE_BYTES_64 = 128 * 64 * 2;  // one 128-row x 64-column 16-bit box = 16 KB

template <int D>
struct FwdCfg {
  static constexpr int CHUNK_COLS = chunk_cols(D);
  static constexpr int CHUNKS = D / CHUNK_COLS;
  static constexpr int CHUNK_BYTES = chunk_bytes(D);
  static constexpr int TILE_BYTES = CHUNKS * CHUNK_BYTES;  // 128 rows x D columns
#ifdef KFA_FWD_STAGES_128
  static constexpr int STAGES = (D > 96) ? KFA_FWD_STAGES_128 : 6;
#else
  static constexpr int STAGES = (D > 96) ? 4 : 6;  // (96: 2 x 24 + 6 x 24 KB)
#endif
  static constexpr int SMEM_TILES = 2 * TILE_BYTES + STAGES * TILE_BYTES;
  static constexpr int SMEM_BYTES = SMEM_TILES + 1024 /*alignment slack*/ + FWD_BAR_BYTES + FWD_HANDOVER_BYTES;
  static constexpr int SMEM_BYTES_LIST = SMEM_BYTES + 2 * TILE_LIST_CAP;  // + the list of visited key tiles
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t TM_S0 = 0, TM_S1 = 128, TM_O0 = 256, TM_O1 = 256 + D;
};

// Keys visible to query row r: [0, key_limit).
__device__ __forceinline__ int key_limit(int r, int P, int Skv) {
  if (P <= 0) return Skv;
  long long lim = (static_cast<long long>(r / P) + 1) * P;
  return lim < Skv ? static_cast<int>(lim) : Skv;
}

// Debug build only (-DKFA_TRACE): CTA 0 of the forward and of the dK / dV kernel records clock64() at its
// hand-offs, per role, key-tile step, part and event; `kfa_trace_read` copies the table to the host.
#ifdef KFA_TRACE
__device__ long long kfa_trace[6][64][2][8];
#define TR(role, j, part, ev) do { if (trace_on && (j) < 64) kfa_trace[role][j][part][ev] = clock64(); } while (0)
#else
#define TR(role, j, part, ev) do {} while (0)
#endif

// First 128-row query tile all of whose rows see every key of the 128-key tile at kv0 (block-causal frame
// P > 0, the key tile complete): tile i is fully visible iff key_limit(128 i) >= kv0 + 128, which is monotone
// in i. Computed once per CTA, so that the key-major loops do no division per step.
__device__ __forceinline__ int first_full_tile(int kv0, int P) {
  const long long t = (static_cast<long long>(kv0) + 128 + P - 1) / P - 1;
  return static_cast<int>((t * P + 127) / 128);
}

// Launch order of the main kernels: the (batch, head) pairs in groups of 8; inside a group tile-major. Under a
// causal mask every head's tiles run from the heaviest to the lightest, so a group's heavy tiles all start
// before its light ones and the launch ends on light tiles (head after head, the last wave would hold
// heavy tiles of the last heads: 4 % of the forward's time at 128 heads, 30 % at 16), while the CTAs that
// run side by side still share the K / V (or Q / dO) of a few heads in L2.
__device__ __forceinline__ void decode_tile(int idx, int n_bh, int n_tiles, int& bh, int& t) {
  constexpr int G = 8;
  const int per_group = G * n_tiles;
  const int g = idx / per_group;
  const int r = idx - g * per_group;
  const int gs = min(G, n_bh - g * G);
  t = r / gs;
  bh = g * G + (r - t * gs);
}

// Walk over the steps of a key-major CTA without a division per step: query tile (relative to the first
// one that sees the keys) and query head of the K / V head's group.
struct StepWalk {
  int rel = 0, g = 0;
  __device__ __forceinline__ void next(int n_per) {
    if (++rel == n_per) {
      rel = 0;
      ++g;
    }
  }
};

template <int D, bool BF16, bool MASKW>
__global__ void __launch_bounds__(FWD_THREADS, 1)
kfa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int CH = Cfg::CHUNKS;
  constexpr int NS = Cfg::STAGES;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base;                        // [half][chunk] 16 KB boxes
  const uint32_t sKV = smem_base + 2 * Cfg::TILE_BYTES;  // [stage][chunk]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::SMEM_TILES);
  // barrier indices
  constexpr int B_QREADY = 0;             // 2
  constexpr int B_KVREADY = 2;            // NS
  constexpr int B_KVFREE = 2 + NS;        // NS
  constexpr int B_SREADY = 2 + 2 * NS;    // 4: [half][part] the 64 score columns of that part are in TMEM
  constexpr int B_PREADY = 6 + 2 * NS;    // 4: [half][part] the 64 keys of P_h of that part are stored (128 arrivals)
  constexpr int B_OFINAL = 10 + 2 * NS;   // 2
  constexpr int B_DRAIN = 12 + 2 * NS;    // 2: [half] everything that half's MMA warp issued has retired
  constexpr int B_PVDONE = 14 + 2 * NS;   // 4: [half][part] that part of O_h += P V has retired
  constexpr int B_ALPHA = 18 + 2 * NS;    // 4: [half][part] the rows' rescale factors are in shared memory (128 arrivals)
  constexpr int B_OREADY = 22 + 2 * NS;   // 4: [half][part] O_h is rescaled for that part (128 arrivals)
  constexpr int N_BARS = 26 + 2 * NS;
  static_assert(N_BARS * 8 + 16 <= FWD_BAR_BYTES, "barrier block too small");
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  // hand-over between the softmax and the correction warpgroups: alpha [half][part][row]
  float* s_alpha = reinterpret_cast<float*>(smem + Cfg::SMEM_TILES + FWD_BAR_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
#ifdef KFA_TRACE
  const bool trace_on = (blockIdx.x == 0) && (lane == 0);
  if (warp == 8) TR(2, 0, 0, 4);
#endif

  // ---- tile decode (groups of heads, tile-major inside), heaviest query tile first when causal ----
  int bh, t;
  decode_tile(blockIdx.x, p.B * p.H, p.n_q_tiles, bh, t);
  const int q_tile = (p.P > 0) ? (p.n_q_tiles - 1 - t) : t;
  const int b = bh / p.H;
  const int h = bh % p.H;
  const int row0 = q_tile * 256;  // relative to the sequence's first row
  int Sq = p.Sq, Skv = p.Skv, q_base = 0, k_base = 0, bc = b;  // bc: batch coordinate in the tensors
  if (p.cu_q != nullptr) {
    q_base = p.cu_q[b];
    Sq = p.cu_q[b + 1] - q_base;
    k_base = p.cu_k[b];
    Skv = p.cu_k[b + 1] - k_base;
    bc = 0;
    if (row0 >= Sq || Skv <= 0) return;  // the whole CTA, before anything is set up
  }

  int n_tiles[2], n_unmasked[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int first = row0 + 128 * hf;
    if (first < Sq) {
      const int last = min(first + 127, Sq - 1);
      n_tiles[hf] = (key_limit(last, p.P, Skv) + 127) / 128;
      n_unmasked[hf] = key_limit(first, p.P, Skv) / 128;
    } else {
      n_tiles[hf] = 0;
      n_unmasked[hf] = 0;
    }
  }
  int n_max = max(n_tiles[0], n_tiles[1]);
  // boolean masks with a tile table: the key tiles this CTA visits, in shared memory
  uint16_t* s_list = reinterpret_cast<uint16_t*>(smem + Cfg::SMEM_TILES + FWD_BAR_BYTES + FWD_HANDOVER_BYTES);
  const bool use_list = MASKW && p.mt != nullptr;

  // ---- setup ----
  if (tid == 0) {
    mbar_init(bar(B_QREADY + 0), 1);
    mbar_init(bar(B_QREADY + 1), 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(bar(B_KVREADY + i), 1);
      mbar_init(bar(B_KVFREE + i), 2);  // one arrival per MMA warp
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar(B_SREADY + i), 1);
      mbar_init(bar(B_PREADY + i), 128);
      mbar_init(bar(B_PVDONE + i), 1);
      mbar_init(bar(B_ALPHA + i), 128);
      mbar_init(bar(B_OREADY + i), 128);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_OFINAL + i), 1);
      mbar_init(bar(B_DRAIN + i), 1);
    }
    // An earlier failure (status word already set): allocate, skip the work, free.
    *s_abort = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(s_tmem), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if constexpr (MASKW) {
    if (use_list && warp == 1) {  // (warp 0 allocates tensor memory meanwhile)
      const int* t0 = p.mt + bc * p.mt_sb + h * p.mt_sh + static_cast<long long>(2 * q_tile) * p.mt_row;
      const bool two = row0 + 128 < Sq;
      int count = 0;
      for (int j0 = 0; j0 < n_max; j0 += 32) {
        const int j = j0 + lane;
        bool seen = false;
        if (j < n_max) seen = (__ldg(t0 + j) | (two ? __ldg(t0 + p.mt_row + j) : 0)) != 0;
        const unsigned m = __ballot_sync(0xffffffffu, seen);
        if (seen) s_list[count + __popc(m & ((1u << lane) - 1u))] = static_cast<uint16_t>(j);
        count += __popc(m);
      }
      if (count == 0) {  // nothing visible at all: one tile still runs, so that the rows get their zeros
        if (lane == 0) s_list[0] = 0;
        count = 1;
      }
      if (lane == 0) s_tmem[2] = static_cast<uint32_t>(count);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  if (warp == 8) TR(2, 0, 0, 5);
  if (use_list) {
    n_max = static_cast<int>(s_tmem[2]);
    n_tiles[0] = n_tiles[0] > 0 ? n_max : 0;
    n_tiles[1] = n_tiles[1] > 0 ? n_max : 0;
  }
  auto tile_of = [&](int it) { return use_list ? static_cast<int>(s_list[it]) : it; };
  const Ctl ctl{s_abort, p.status};
  const bool dead = (*s_abort != 0);

  // Each role sets its register budget first (the kernel starts with 128 per thread).
  if (dead) {
    // nothing to do
  } else if (warp == 15) {
    reg_budget<FWD_REGS_ISSUE>();
  } else if (warp == 13) {
    // =========================== TMA producer ===========================
    reg_budget<FWD_REGS_ISSUE>();
    if (lane == 0) {
      prefetch_tensormap(&tmQ);
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmV);
      for (int hf = 0; hf < 2; ++hf) {
        if (n_tiles[hf] == 0) continue;
        mbar_expect_tx(bar(B_QREADY + hf), Cfg::TILE_BYTES);
        for (int ch = 0; ch < CH; ++ch)
          tma_load_4d(sQ + (hf * CH + ch) * Cfg::CHUNK_BYTES, &tmQ, bar(B_QREADY + hf), ch * Cfg::CHUNK_COLS,
                      q_base + row0 + 128 * hf, h, bc);
      }
      int armed[NS];  // last use index armed per stage (for the drain on abort)
      for (int i = 0; i < NS; ++i) armed[i] = -1;
      bool ok = true;
      for (int idx = 0; idx < 2 * n_max && ok; ++idx) {
        const int j = tile_of(idx >> 1);
        const int stage = idx % NS;
        const int use = idx / NS;
        if (use > 0) ok = mbar_wait(bar(B_KVFREE + stage), (use - 1) & 1, ctl, 1);
        if (!ok) break;
        mbar_expect_tx(bar(B_KVREADY + stage), Cfg::TILE_BYTES);
        const CUtensorMap* map = (idx & 1) ? &tmV : &tmK;
        for (int ch = 0; ch < CH; ++ch)
          tma_load_4d(sKV + (stage * CH + ch) * Cfg::CHUNK_BYTES, map, bar(B_KVREADY + stage), ch * Cfg::CHUNK_COLS,
                      k_base + j * 128, h / p.group, bc);
        armed[stage] = use;
      }
      if (!ok) {
        // Aborting: let the copies already in flight land before the CTA gives up its smem.
        for (int hf = 0; hf < 2; ++hf)
          if (n_tiles[hf] > 0) mbar_drain(bar(B_QREADY + hf), 0);
        for (int i = 0; i < NS; ++i)
          if (armed[i] >= 0) mbar_drain(bar(B_KVREADY + i), armed[i] & 1);
      }
    }
  } else if (warp == 12 || warp == 14) {
    // =========================== MMA issue ===========================
    // One warp per half (12: half 0, 14: half 1): the two halves' chains are independent, and two issuing
    // warps keep the tensor core fed while one of them sits in its waits. The whole warp runs this role
    // converged; one elected lane issues the tcgen05 instructions. A K / V stage is free again once BOTH
    // warps' instructions that read it have retired (a commit counts only the committing thread's own).
    reg_budget<FWD_REGS_ISSUE>();
    {
      const int hf = (warp - 12) >> 1;
      const bool lead = elect_one();
      constexpr uint32_t IDESC_S = make_idesc(BF16, false, 128, FWD_PART_KEYS);
      constexpr uint32_t IDESC_O = make_idesc(BF16, true, 128, D);
      constexpr uint32_t HI = sdesc_hi_for(D);
      const uint32_t tmS = tmem + (hf ? Cfg::TM_S1 : Cfg::TM_S0);
      const uint32_t tmO = tmem + (hf ? Cfg::TM_O1 : Cfg::TM_O0);
      const uint32_t q_lo = sdesc_lo(sQ + hf * Cfg::TILE_BYTES, 16);
      const int nt = n_tiles[hf];
      bool ok = true;

      // S_h of the 64 keys of one part (rows 64 part .. of the K tile) into columns 64 part .. of S_h
      auto issue_S = [&](int stage, int part) {
        const uint32_t k_lo = sdesc_lo(sKV + stage * Cfg::TILE_BYTES + part * (FWD_PART_KEYS * 2 * Cfg::CHUNK_COLS), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = kstep_bytes(D, kk) >> 4;
          umma_ss_lead(lead, tmS + FWD_PART_KEYS * part, q_lo + off, k_lo + off, IDESC_S, kk > 0 ? 1u : 0u, HI);
        }
      };
      // O_h += P V over the 64 keys of one part; its 16-bit P sits in the first 32 columns of the part
      auto issue_PV = [&](int stage, bool acc, int part) {
        const uint32_t v_lo = sdesc_lo(sKV + stage * Cfg::TILE_BYTES, Cfg::CHUNK_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < FWD_PART_KEYS / 16; ++k4) {
          const int kk = part * (FWD_PART_KEYS / 16) + k4;
          umma_ts_lead(lead, tmO, tmS + FWD_PART_KEYS * part + k4 * 8, v_lo + (kstep_rows_bytes(D, kk) >> 4), IDESC_O,
                       (acc || kk > 0) ? 1u : 0u, HI);
        }
      };
      auto kv_wait = [&](int idx) {
        return mbar_wait_warp(bar(B_KVREADY + idx % NS), (idx / NS) & 1, ctl, 2);
      };

      // S(0), both parts
      ok = kv_wait(0);
      if (ok && nt > 0) {
        ok = mbar_wait_warp(bar(B_QREADY + hf), 0, ctl, 3);
        if (ok) {
          tc_fence_after();
          for (int part = 0; part < FWD_PARTS; ++part) {
            issue_S(0, part);
            umma_commit_lead(lead, bar(B_SREADY + 2 * hf + part));
          }
        }
      }
      if (ok) umma_commit_lead(lead, bar(B_KVFREE + 0));

      // Per key tile and 64-key part: O_h += P V of the part (once its P is stored and O_h carries the
      // part's rescale), then the next tile's scores of the same part overwrite it. The other part of S_h
      // is untouched meanwhile, so the softmax of one part runs while the tensor core works on the other.
      for (int j = 0; j < n_max && ok; ++j) {
        const int iv = 2 * j + 1;  // V_j
        const int ik = 2 * j + 2;  // K_{j+1}
        const bool more = (j + 1 < n_max);
        ok = kv_wait(iv);
        if (!ok) break;
        if (more) {
          ok = kv_wait(ik);
          if (!ok) break;
        }
        for (int part = 0; part < FWD_PARTS && ok; ++part) {
          if (j < nt) {
            TR(3 + 2 * hf, j, part, 0);
            ok = mbar_wait_warp(bar(B_PREADY + 2 * hf + part), j & 1, ctl, 4);
            TR(3 + 2 * hf, j, part, 1);
            if (ok) ok = mbar_wait_warp(bar(B_OREADY + 2 * hf + part), j & 1, ctl, 8);
            if (!ok) break;
            TR(3 + 2 * hf, j, part, 2);
            tc_fence_after();
            issue_PV(iv % NS, j > 0, part);
            umma_commit_lead(lead, bar(B_PVDONE + 2 * hf + part));
            if (part == FWD_PARTS - 1 && j == nt - 1) umma_commit_lead(lead, bar(B_OFINAL + hf));
            TR(3 + 2 * hf, j, part, 3);
          }
          if (more && j + 1 < nt) {
            issue_S(ik % NS, part);
            umma_commit_lead(lead, bar(B_SREADY + 2 * hf + part));
            TR(3 + 2 * hf, j, part, 4);
          }
        }
        if (ok) {
          umma_commit_lead(lead, bar(B_KVFREE + iv % NS));
          if (more) umma_commit_lead(lead, bar(B_KVFREE + ik % NS));
        }
      }
      // Everything issued has to retire before TMEM is freed.
      umma_commit_lead(lead, bar(B_DRAIN + hf));
      mbar_drain(bar(B_DRAIN + hf), 0);
    }
  } else if (warp >= 8) {
    // =========================== correction: rescale of O ===========================
    // Thread t <-> row t of BOTH halves. For every (half, part) in the order the MMA warp consumes them:
    // take the rows' factors alpha = exp2((m_old - m_new) c) from the softmax warpgroup, multiply O_h by
    // them if any row of the warp moved its max (exact; bit-identical to always multiplying), release the
    // part's P V. This runs while the softmax warpgroup computes the part's exponentials.
    reg_budget<FWD_REGS_CORRECTION>();
    const int r_in = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tOh[2] = {tmem + Cfg::TM_O0 + lane_base, tmem + Cfg::TM_O1 + lane_base};
    bool ok = true;
    for (int j = 0; j < n_max && ok; ++j) {
      for (int part = 0; part < FWD_PARTS && ok; ++part) {
        for (int hf = 0; hf < 2; ++hf) {
          if (j >= n_tiles[hf]) continue;
          if (warp == 8) TR(2 + 2 * hf, j, part, 0);
          ok = mbar_wait_warp(bar(B_ALPHA + 2 * hf + part), j & 1, ctl, 9);
          if (!ok) break;
          if (warp == 8) TR(2 + 2 * hf, j, part, 1);
          const float alpha = s_alpha[(2 * hf + part) * 128 + r_in];
          if ((j > 0 || part > 0) && !__all_sync(0xffffffffu, alpha == 1.0f)) {
            // every part of O_h += P V issued so far has to have retired (the barrier of the previous part
            // cannot be two phases ahead: the part after the next needs this release)
            const int prev = FWD_PARTS * j + part - 1;
            ok = mbar_wait_warp(bar(B_PVDONE + 2 * hf + (prev % FWD_PARTS)), (prev / FWD_PARTS) & 1, ctl, 7);
            if (!ok) break;
            tc_fence_after();
            const float2 a2 = make_float2(alpha, alpha);
            constexpr int W = col_step(D);
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += W) {
              float2 o[W / 2];
              tmem_ldw<W>(tOh[hf] + c0, reinterpret_cast<uint32_t*>(o));
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < W / 2; ++i) o[i] = __fmul2_rn(o[i], a2);
              tmem_stw<W>(tOh[hf] + c0, reinterpret_cast<const uint32_t*>(o));
            }
            tmem_wait_st();
          }
          tc_fence_before();
          mbar_arrive(bar(B_OREADY + 2 * hf + part));
          if (warp == 8) TR(2 + 2 * hf, j, part, 2);
        }
      }
    }
  } else {
    // =========================== softmax ===========================
    reg_budget<FWD_REGS_SOFTMAX>();
    const int hf = warp >> 2;
    const int r_in = tid & 127;
    const int row = row0 + 128 * hf + r_in;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + (hf ? Cfg::TM_S1 : Cfg::TM_S0) + lane_base;
    const int nt = n_tiles[hf];
    const int nu = n_unmasked[hf];
    const int my_limit = key_limit(min(row, Sq - 1), p.P, Skv);
    const float c = p.c;

    float m = -INFINITY;
    float l = 0.f;
    bool ok = true;
    bool s_probe = false;  // an early test of the next part's score barrier (see mbar_wait_warp_probed)
    // boolean mask: this row's words, one 16-byte load per key tile, fetched a tile ahead
    const uint4* mrow = nullptr;
    uint4 mnext = make_uint4(0u, 0u, 0u, 0u);
    if constexpr (MASKW) {
      mrow = reinterpret_cast<const uint4*>(p.mw + bc * p.mw_sb + h * p.mw_sh +
                                            static_cast<long long>(min(row, Sq - 1)) * p.mw_row);
      if (nt > 0) mnext = __ldg(mrow + tile_of(0));
    }
    for (int j = 0; j < nt; ++j) {  // j counts visited tiles (tile_of(j) is the key tile)
      uint32_t mbits[4] = {mnext.x, mnext.y, mnext.z, mnext.w};
      bool apply_bits = false;
      if constexpr (MASKW) {
        if (j + 1 < nt) mnext = __ldg(mrow + tile_of(j + 1));
        apply_bits = !__all_sync(0xffffffffu, (mbits[0] & mbits[1] & mbits[2] & mbits[3]) == 0xffffffffu);
      }
      const bool masked = (j >= nu);
      // The tile's 128 keys are handled as two parts of 64 with their own score columns, so that the
      // tensor core refills one part while this thread works on the other.
#pragma unroll
      for (int part = 0; part < FWD_PARTS; ++part) {
        constexpr int PK = FWD_PART_KEYS;
        if ((warp & 3) == 0) TR(hf, j, part, 0);
        ok = mbar_wait_warp_probed(s_probe, bar(B_SREADY + 2 * hf + part), j & 1, ctl, 5);
        if (!ok) break;
        if ((warp & 3) == 0) TR(hf, j, part, 1);
        tc_fence_after();
        const uint32_t tSp = tS + PK * part;
        const int lim = my_limit - j * 128 - PK * part;
        float s[PK];
#pragma unroll
        for (int c0 = 0; c0 < PK; c0 += 32) tmem_ld32(tSp + c0, reinterpret_cast<uint32_t*>(s + c0));
        tmem_wait_ld();
        if ((warp & 3) == 0) TR(hf, j, part, 2);
        if constexpr (MASKW) {
          if (apply_bits) {
#pragma unroll
            for (int i = 0; i < PK; ++i)
              if (!((mbits[(PK / 32) * part + (i >> 5)] >> (i & 31)) & 1u)) s[i] = -INFINITY;
          }
        } else if (masked) {
#pragma unroll
          for (int i = 0; i < PK; ++i)
            if (i >= lim) s[i] = -INFINITY;
        }
        float mx0 = fmaxf(s[0], s[1]), mx1 = fmaxf(s[2], s[3]), mx2 = fmaxf(s[4], s[5]), mx3 = fmaxf(s[6], s[7]);
#pragma unroll
        for (int i = 8; i < PK; i += 8) {  // pairs of maxima: three-input max instructions
          mx0 = fmaxf(mx0, fmaxf(s[i], s[i + 1]));
          mx1 = fmaxf(mx1, fmaxf(s[i + 2], s[i + 3]));
          mx2 = fmaxf(mx2, fmaxf(s[i + 4], s[i + 5]));
          mx3 = fmaxf(mx3, fmaxf(s[i + 6], s[i + 7]));
        }
        const float m_new = fmaxf(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)), m);
        // A row that has seen no key yet (boolean masks only) shifts by 0: its exponents stay -inf, P = 0.
        const float m_shift = (MASKW && m_new == -INFINITY) ? 0.f : m_new;
        // Shift first, then scale: the largest exponent of the row is exactly 0.
        const float alpha = ex2(__fmul_rn(__fsub_rn(m, m_shift), c));
        m = m_new;
        // hand the factor to the correction warpgroup: it rescales O_h while the exponentials below run
        s_alpha[(2 * hf + part) * 128 + r_in] = alpha;
        mbar_arrive(bar(B_ALPHA + 2 * hf + part));
        if ((warp & 3) == 0) TR(hf, j, part, 3);
        // At head dims up to 64 (short MMAs) the scores of the part after this one are usually there already:
        // tested now, settled after the exponentials (-7 % at D=64; at D=128 the early test mostly fails and
        // costs 1 %).
        if constexpr (D <= 64) {
          const int npart = (part + 1) % FWD_PARTS;
          const int nj = (part + 1 == FWD_PARTS) ? j + 1 : j;
          s_probe = (nj < nt) && mbar_test(bar(B_SREADY + 2 * hf + npart), nj & 1);
        }
        // ---- the exponentials, 64 keys at a time (their P goes to tensor memory as soon as it is packed) ----
        const float2 neg_m = make_float2(-m_shift, -m_shift);
        const float2 c2 = make_float2(c, c);
        float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
        const float2* s2 = reinterpret_cast<const float2*>(s);
        uint32_t pk[PK / 2];
        {
#pragma unroll
          for (int i = 0; i < PK / 2; i += 2) {
            const float2 x0 = __fmul2_rn(__fadd2_rn(s2[i], neg_m), c2);
            const float2 x1 = __fmul2_rn(__fadd2_rn(s2[i + 1], neg_m), c2);
            const float2 p0 = make_float2(ex2(x0.x), ex2(x0.y));
            const float2 p1 = make_float2(ex2(x1.x), ex2(x1.y));
            la = __fadd2_rn(la, p0);
            lb = __fadd2_rn(lb, p1);
            pk[i] = pack16<BF16>(p0.x, p0.y);
            pk[i + 1] = pack16<BF16>(p1.x, p1.y);
          }
        }
#pragma unroll
        for (int c0 = 0; c0 < PK / 2; c0 += 32) tmem_st32(tSp + c0, pk + c0);  // P over the score columns already in registers
        if ((warp & 3) == 0) TR(hf, j, part, 4);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(B_PREADY + 2 * hf + part));
        if ((warp & 3) == 0) TR(hf, j, part, 5);
        l = l * alpha + ((la.x + la.y) + (lb.x + lb.y));
      }
      if (!ok) break;
    }
    // ---- epilogue: each softmax warpgroup writes its own half (the rows' m and l are in its registers) ----
    if (ok && nt > 0) ok = mbar_wait_warp(bar(B_OFINAL + hf), 0, ctl, 6);
    if (ok && nt > 0) {
      if ((warp & 3) == 0) TR(2, 0, 1, 4 + hf);
      tc_fence_after();
      const uint32_t tO = tmem + (hf ? Cfg::TM_O1 : Cfg::TM_O0) + lane_base;
      if (p.mode != 0) {
        // Partial result of a context-parallel step: the unnormalised fp32 O with its (m, l) goes to
        // (mode 1), or is merged into (mode 2), the carry in global memory. Merging keeps the two
        // statistics apart and shifts both sides to the common row max before anything is rounded.
        const bool valid = row < Sq;
        const long long bhl = static_cast<long long>(b) * p.H + h;
        float* mlp = p.ml + bhl * p.ml_sh + row;
        float* arow = p.o_acc + bhl * p.oa_sh + static_cast<long long>(row) * D;
        float a_new = 1.0f, a_old = 0.0f;
        if (p.mode == 2 && valid) {
          const float m_old = mlp[0], l_old = mlp[p.ml_plane];
          const float m_tot = fmaxf(m, m_old);
          a_new = ex2(__fmul_rn(__fsub_rn(m, m_tot), c));
          a_old = ex2(__fmul_rn(__fsub_rn(m_old, m_tot), c));
          l = l * a_new + l_old * a_old;
          m = m_tot;
        }
        constexpr int W = col_step(D);
#pragma unroll
        for (int cc = 0; cc < D; cc += W) {
          float o[W];
          tmem_ldw<W>(tO + cc, reinterpret_cast<uint32_t*>(o));
          tmem_wait_ld();
          if (valid) {
#pragma unroll
            for (int i = 0; i < W; i += 4) {
              float4 w = make_float4(o[i] * a_new, o[i + 1] * a_new, o[i + 2] * a_new, o[i + 3] * a_new);
              if (p.mode == 2) {
                const float4 old = *reinterpret_cast<const float4*>(arow + cc + i);
                w.x = fmaf(old.x, a_old, w.x);
                w.y = fmaf(old.y, a_old, w.y);
                w.z = fmaf(old.z, a_old, w.z);
                w.w = fmaf(old.w, a_old, w.w);
              }
              *reinterpret_cast<float4*>(arow + cc + i) = w;
            }
          }
        }
        if (valid) {
          mlp[0] = m;
          mlp[p.ml_plane] = l;
        }
      } else {
        float inv = 1.0f / l;
        float log2_l = log2f(l);
        if (MASKW && l == 0.f) {  // a row with no visible key: output 0, m = +inf, so every P of its backward is 0
          inv = 0.f;
          m = INFINITY;
          log2_l = 0.f;
        }
        const bool valid = row < Sq;
        uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                        2 * (bc * p.o_sb + h * p.o_sh + static_cast<long long>(q_base + row) * p.o_ss);
        constexpr int W = col_step(D);
#pragma unroll
        for (int cc = 0; cc < D; cc += W) {
          float o[W];
          tmem_ldw<W>(tO + cc, reinterpret_cast<uint32_t*>(o));
          tmem_wait_ld();
          if (valid) {
#pragma unroll
            for (int i = 0; i < W; i += 8) {
              uint4 w;
              w.x = pack16<BF16>(o[i] * inv, o[i + 1] * inv);
              w.y = pack16<BF16>(o[i + 2] * inv, o[i + 3] * inv);
              w.z = pack16<BF16>(o[i + 4] * inv, o[i + 5] * inv);
              w.w = pack16<BF16>(o[i + 6] * inv, o[i + 7] * inv);
              *reinterpret_cast<uint4*>(orow + 2 * (cc + i)) = w;
            }
          }
        }
        if (valid) {
          float* lse = p.lse + (static_cast<long long>(bc) * p.H + h) * 2 * p.Sq + q_base;
          lse[row] = m;
          lse[p.Sq + row] = log2_l;
        }
      }
    }
  }

  // ---- teardown (every thread gets here, also after an abort) ----
  if (warp == 8) TR(2, 1, 0, 4);
  tc_fence_before();
  __syncthreads();
  if (warp == 8) TR(2, 1, 0, 5);
  if (*s_abort) {  // gave up (or an earlier kernel did): the rows of this CTA read as NaN
    const int r1 = min(row0 + 256, Sq);
    const long long bhl = static_cast<long long>(b) * p.H + h;
    if (p.mode == 0) {
      fill_rows_nan16(reinterpret_cast<uint8_t*>(p.o) + 2 * (bc * p.o_sb + h * p.o_sh), p.o_ss, q_base + row0, q_base + r1, D);
      float* lse = p.lse + (static_cast<long long>(bc) * p.H + h) * 2 * p.Sq + q_base;
      fill_nan32(lse + row0, r1 - row0);
      fill_nan32(lse + p.Sq + row0, r1 - row0);
    } else {
      fill_nan32(p.ml + bhl * p.ml_sh + row0, r1 - row0);
      fill_nan32(p.ml + bhl * p.ml_sh + p.ml_plane + row0, r1 - row0);
    }
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

}  // namespace kfa
