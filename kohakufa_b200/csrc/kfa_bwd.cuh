// Attention backward for sm_100a, as three kernels:
//
//   kfa_bwd_prepare_kernel   delta = rowsum(fp32(dO) * fp32(O)); packs (-m, -log2 l, -delta) per
//                            128-row query tile, padded rows get -m = -inf so their P is 0
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
// Roles in both main kernels (320 threads):
//   warps 0-3  columns 0-63 of every 128x128 score tile     warp 8  MMA issue (converged, one lane issues)
//   warps 4-7  columns 64-127                               warp 9  TMA producer
// Thread t of a warpgroup owns TMEM lane t (a key row in the dK/dV kernel, a query row in the dQ
// kernel). A step has two compute phases, P from S and then dS from dP, each followed by an MMA that
// consumes the 16-bit result straight from TMEM (P^T / dS^T overwrite the S^T / dP^T columns they
// came from). The MMA warp interleaves the four (three) MMAs of consecutive steps,
//   dK/dV:  dV(i)  S^T(i+1)  dK(i)  dP^T(i+1)          dQ:  S(j+1)  dQ(j)  dP(j+1)   (D > 64: S(j+1)  dP(j+1)  dQ(j),
//                                                          with dS in columns of its own: see BwdCfg::DS_OWN)
// so that while the warpgroups compute one phase the tensor core always has another MMA to run, and
// every smem x smem MMA is a full 128-column one (64-column ones run at 2/3 rate on this part).
//
// Numerics kept from the reference (docs/precision.md:27-34, 90-114; bwd.py:1036-1043, 1083-1086):
//   * P = exp2(fma(S - m, c, -log2 l)) from the two separate statistics, never a fused lse;
//   * dS, not scale * dS, is rounded to 16 bits and fed to the MMAs; scale multiplies the fp32 dK and
//     dQ accumulators afterwards;
//   * padded keys and hidden (key, query) pairs get P = 0 exactly; padded query rows carry -m = -inf.
// One difference: dS = (dP - delta) * P uses the fp32 P, not the 16-bit rounded one (one rounding less).
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
  const float* stats;  // [B*H, n_q128, 3, 128]: -m, -log2 l, -delta
  int B, H, Sq, Skv;
  int Hkv, group;  // K / V heads; query heads per K / V head (H = Hkv * group)
  int P;
  float c;      // scale * log2(e)
  float scale;  // applied to fp32 dK and dQ
  int n_q128, n_k128;
  int* status;
  long long stats_sh;  // floats between the statistics of consecutive (b, h): n_q128 * 384 unless a slice
  // Context-parallel steps (acc_mode != 0): the scaled fp32 gradients are stored to (1) or added to
  // (2) fp32 accumulators instead of being rounded to 16 bits. Row r of (b, h) at ptr + (b*H+h)*sh + r*D.
  int acc_mode;
  float* dq32;
  long long dq32_sh;
  float* dk32;
  long long dk32_sh;
  float* dv32;
  long long dv32_sh;
  // Packed variable-length batches (cu_q != nullptr): tensors [1, H, T, D], sequence b (of B) owns query
  // rows cu_q[b] .. cu_q[b + 1] and key rows cu_k[b] .. cu_k[b + 1]. Sq, Skv are then the tensors' row
  // counts and n_q128 / n_k128 the tile counts of the longest sequence (they size the grid and the
  // statistics, whose tiles are numbered from each sequence's first row).
  const int* cu_q;
  const int* cu_k;
  // Boolean mask (kernels instantiated with MASKW), bit set = visible. mw: 32 keys per word along query
  // rows (row r of (b, h) at mw + b * mw_sb + h * mw_sh + r * mw_row), read by the dQ kernel; mwt: 32
  // queries per word along key rows, read by the dK / dV kernel. Strides of 0 broadcast; four words per
  // 128-wide tile; zero bits past the ends.
  const int* mw;
  long long mw_sb, mw_sh;
  int mw_row;
  const int* mwt;
  long long mwt_sb, mwt_sh;
  int mwt_row;
  // Optional with a mask: nonzero = some bit of the (128 queries x 128 keys) tile is set; tile (qt, kt) of
  // (b, h) at mt + b * mt_sb + h * mt_sh + qt * mt_row + kt. Tile pairs without a visible pair are skipped.
  const int* mt;
  long long mt_sb, mt_sh;
  int mt_row;
};

struct PrepParams {
  const void* o;
  long long o_sb, o_sh, o_ss;
  const void* dout;
  long long do_sb, do_sh, do_ss;
  const float* lse;  // [B, H, 2, Sq]
  float* stats;      // [B*H, n_q128, 3, 128]
  int B, H, Sq, n_q128;
  const int* cu_q;  // packed variable-length batches: see BwdParams
  // Fused backward only (else nullptr): the fp32 dQ accumulator, whole 128-row tiles of D floats per
  // (batch, head); every CTA zero-fills the tile of its rows.
  float* dq_acc;
};

// ---------------------------------------------------------------------------------------
// prepare: HBM-bound; D / 8 lanes per row (rounded up to a power of two), 16-byte loads.
// ---------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(128) kfa_bwd_prepare_kernel(const PrepParams p) {
  constexpr int VECS = D / 8;                                                      // 16-byte pieces of a row
  constexpr int LPR = VECS <= 2 ? 2 : (VECS <= 4 ? 4 : (VECS <= 8 ? 8 : 16));      // lanes per row (a power of two)
  constexpr int RPW = 32 / LPR;                                                    // rows per warp pass
  const int tile = blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, vec = lane % LPR;
  int Sq = p.Sq, bc = b;
  long long q_base = 0;
  if (p.cu_q != nullptr) {
    q_base = p.cu_q[b];
    Sq = p.cu_q[b + 1] - static_cast<int>(q_base);
    bc = 0;
  }
  const uint8_t* ob = reinterpret_cast<const uint8_t*>(p.o) + 2 * (bc * p.o_sb + h * p.o_sh + q_base * p.o_ss);
  const uint8_t* gb = reinterpret_cast<const uint8_t*>(p.dout) + 2 * (bc * p.do_sb + h * p.do_sh + q_base * p.do_ss);
  float* st = p.stats + (static_cast<long long>(bh) * p.n_q128 + tile) * 384;
  const float* lse = p.lse + (static_cast<long long>(bc) * p.H + h) * 2 * p.Sq + q_base;
  if (p.dq_acc != nullptr) {
    float4* acc = reinterpret_cast<float4*>(p.dq_acc + (static_cast<long long>(bh) * p.n_q128 + tile) * (128 * D));
#pragma unroll 4
    for (int i = threadIdx.x; i < 128 * D / 4; i += 128) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int r0 = warp * 32; r0 < warp * 32 + 32; r0 += RPW) {
    const int r_in = r0 + sub;
    const int row = tile * 128 + r_in;
    float acc = 0.f;
    if (row < Sq && vec < VECS) {
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
      const bool valid = row < Sq;
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
  static constexpr int CHUNK_COLS = chunk_cols(D);
  static constexpr int CHUNKS = D / CHUNK_COLS;
  static constexpr int CHUNK_BYTES = chunk_bytes(D);
  static constexpr int TILE_BYTES = CHUNKS * CHUNK_BYTES;  // 128 rows x D columns
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t TM_S = 0, TM_DP = 128, TM_ACC0 = 256, TM_ACC1 = 256 + D;
  // dQ kernel at D > 64: the 16-bit dS gets two buffers of 64 columns of its own (dQ ends at 256 + D <= 384), so
  // that dP(j+1) is issued as soon as the warpgroups hold dP(j) instead of after dQ(j): the step is no longer
  // the loop dS(j-1) -> dQ(j-1), dP(j) -> dS(j) through the tensor core (C3: 2.67 -> 2.57 ms). At D <= 64, where
  // the two products are short, dS stays over the dP columns (own columns: 0.564 -> 0.582 ms at C4's shape).
  static constexpr bool DS_OWN = (D > 64);
  static constexpr uint32_t TM_DS = 384;
  // dK/dV kernel: K, V resident; ring of (Q_i, dO_i, stats_i) slots.
  static constexpr int KV_SLOTS = (D > 96) ? 2 : 3;
  static constexpr int KV_SLOT_BYTES = 2 * TILE_BYTES + 2048;  // stats padded to keep 1 KB alignment
  static constexpr int KV_SMEM_TILES = 2 * TILE_BYTES + KV_SLOTS * KV_SLOT_BYTES;
  static constexpr int KV_SMEM_BYTES = KV_SMEM_TILES + 1024 + 256;
  static constexpr int KV_LIST_CAP = 2048;  // (query head, query tile) steps a masked CTA can list
  static constexpr int KV_SMEM_BYTES_LIST = KV_SMEM_BYTES + 4 * KV_LIST_CAP;
  // dQ kernel: Q, dO resident; K_j and V_j through rings of their own. K_j is read by S(j) and, a step
  // later, by dQ(j); V_j only by dP(j): three K buffers and two V buffers let the copy of tile j + 2
  // start a whole step before it is needed (with K and V sharing two slots it could start only when
  // dQ(j) had retired, and the tensor core waited for the copy at every step).
  static constexpr int NK = (D > 96) ? 3 : 4;
  static constexpr int NV = (D > 96) ? 2 : 3;
  static constexpr int Q_SMEM_TILES = (2 + NK + NV) * TILE_BYTES;
  static constexpr int Q_SMEM_BYTES = Q_SMEM_TILES + 1024 + 256;
  static constexpr int Q_LIST_CAP = (D > 96) ? 768 : 1024;  // key tiles a masked CTA can list (what fits)
  static constexpr int Q_SMEM_BYTES_LIST = Q_SMEM_BYTES + 2 * Q_LIST_CAP;
};

// Issue helpers for the MMA warp (converged; `lead` is true in the one lane that issues). Operand
// tiles are swizzled [128 rows][C] boxes, D / C of them one after the other (C = chunk_cols(D));
// descriptors are passed as their low words (see sdesc_lo).
// acc[128 x 128] = A[128 rows, D] * B[128 rows, D]^T, contraction over D.
template <int D>
__device__ __forceinline__ void issue_kmajor_n128(bool lead, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                  uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const uint32_t off = kstep_bytes(D, kk) >> 4;
    umma_ss_lead(lead, d_tmem, a_lo + off, b_lo + off, idesc, kk > 0 ? 1u : 0u, sdesc_hi_for(D));
  }
}
// acc[128 x D] (+)= A16[128 x 128] * B[128 rows, D], contraction over B's rows (MN-major B, leading
// offset = one 16 KB box). The 16-bit A operand sits in TMEM as two 32-column pieces: contraction
// indices 0-63 at a_tmem, 64-127 at a_tmem + 64 (where the two warpgroups wrote their halves).
template <int D>
__device__ __forceinline__ void issue_tmemA_k128(bool lead, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                                 uint32_t idesc, bool acc) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    umma_ts_lead(lead, d_tmem, a_tmem + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8), b_lo + (kstep_rows_bytes(D, kk) >> 4), idesc,
                 (acc || kk > 0) ? 1u : 0u, sdesc_hi_for(D));
}

// The same with the 16-bit A operand as ONE piece of 64 columns (contraction indices 0-127 at a_tmem .. + 63).
template <int D>
__device__ __forceinline__ void issue_tmemA_k128_packed(bool lead, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                                        uint32_t idesc, bool acc) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    umma_ts_lead(lead, d_tmem, a_tmem + kk * 8, b_lo + (kstep_rows_bytes(D, kk) >> 4), idesc, (acc || kk > 0) ? 1u : 0u,
                 sdesc_hi_for(D));
}

// The same for half of the contraction: k-steps 2 * part, 2 * part + 1 of each warpgroup's piece
// (the first or the second 32 of its 64 contraction indices).
template <int D>
__device__ __forceinline__ void issue_tmemA_k64(bool lead, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                                uint32_t idesc, bool acc, int part) {
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    const int kk = (x >> 1) * 4 + 2 * part + (x & 1);
    umma_ts_lead(lead, d_tmem, a_tmem + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8), b_lo + (kstep_rows_bytes(D, kk) >> 4), idesc,
                 (acc || x > 0 || part > 0) ? 1u : 0u, sdesc_hi_for(D));
  }
}

// Stores (add = false) or adds (add = true) a row of an fp32 accumulator times mul to fp32 memory.
template <int W = 32>
__device__ __forceinline__ void store_acc_row_f32(uint32_t taddr, int col0, int ncols, float mul, float* grow,
                                                  bool valid, bool add) {
  for (int cc = col0; cc < col0 + ncols; cc += W) {
    float o[W];
    tmem_ldw<W>(taddr + cc, reinterpret_cast<uint32_t*>(o));
    tmem_wait_ld();
    if (valid) {
#pragma unroll
      for (int i = 0; i < W; i += 4) {
        float4 w = make_float4(o[i] * mul, o[i + 1] * mul, o[i + 2] * mul, o[i + 3] * mul);
        if (add) {
          const float4 old = *reinterpret_cast<const float4*>(grow + cc + i);
          w.x += old.x;
          w.y += old.y;
          w.z += old.z;
          w.w += old.w;
        }
        *reinterpret_cast<float4*>(grow + cc + i) = w;
      }
    }
  }
}

// Writes a row of an fp32 accumulator (TMEM columns [col0, col0 + ncols)) times mul as 16-bit.
template <bool BF16, int W = 32>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, int col0, int ncols, float mul, uint8_t* grow,
                                              bool valid) {
  for (int cc = col0; cc < col0 + ncols; cc += W) {
    float o[W];
    tmem_ldw<W>(taddr + cc, reinterpret_cast<uint32_t*>(o));
    tmem_wait_ld();
    if (valid) {
#pragma unroll
      for (int i = 0; i < W; i += 8) {
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

// P^T and dS^T in the dK / dV kernel. The per-query statistics (-m at st[0..], -log2 l at st[128..],
// -delta at st[256..], in shared memory) belong to COLUMNS of the transposed tile, so every thread
// needs them for every column it touches. With one TMEM lane (key) per thread that is all 64 columns
// of its warpgroup: 192 floats per thread and step, whose broadcast loads cost about 1000 shared-memory
// cycles per step on top of the 1500 the tensor core's operands and 500 the TMA need, and shared
// memory, not the tensor core, bounds the kernel. The fragment shape (tcgen05.ld.16x256b) gives a thread
// 4 keys x 16 queries instead: a quarter of the statistics, as 8-byte loads shared by 8 lanes.
//
// Element order of sv / pr / the packed words: index 16 * half + 2 * j + sel is the column pair
// 8j + 2(lane % 4), +1 of key row (lane / 4 + 8 * sel) of the warp's 16-lane half `half`.
//   P = exp2(fma(S - m, c, -log2 l)), kept in fp32 (pr) and packed to 16 bits (pk).
// MASKED: a pair whose query index is below the key's first visible query (qmin[2 * half + sel]) gets P = 0.
// J0: the four column blocks J0 .. J0 + 3 (32 of the warpgroup's 64 queries) are done per call.
template <bool BF16, bool MASKED, int J0>
__device__ __forceinline__ void p_frag(const float2* sv, const float* st, float2 c2, int q_first, const int* qmin,
                                       float2* pr, uint32_t* pk) {
#pragma unroll
  for (int j = J0; j < J0 + 4; ++j) {
    const float2 nm = *reinterpret_cast<const float2*>(st + 8 * j);
    const float2 nl = *reinterpret_cast<const float2*>(st + 128 + 8 * j);
#pragma unroll
    for (int e = 0; e < 4; ++e) {  // e = 2 * half + sel
      const int idx = 16 * (e >> 1) + 2 * j + (e & 1);
      const float2 x = __ffma2_rn(__fadd2_rn(sv[idx], nm), c2, nl);
      float2 pv = make_float2(ex2(x.x), ex2(x.y));
      if constexpr (MASKED) {
        if (q_first + 8 * j < qmin[e]) pv.x = 0.f;
        if (q_first + 8 * j + 1 < qmin[e]) pv.y = 0.f;
      }
      pr[idx] = pv;
      pk[idx] = pack16<BF16>(pv.x, pv.y);
    }
  }
}
// The same under a boolean mask: w[e] holds the two words (64 queries of this warpgroup) of key row e;
// a pair whose bit is clear gets P = 0. col0 = this thread's first column inside every block of 8.
template <bool BF16, int J0>
__device__ __forceinline__ void p_frag_bits(const float2* sv, const float* st, float2 c2, const uint2* w, int col0,
                                            float2* pr, uint32_t* pk) {
#pragma unroll
  for (int j = J0; j < J0 + 4; ++j) {
    const float2 nm = *reinterpret_cast<const float2*>(st + 8 * j);
    const float2 nl = *reinterpret_cast<const float2*>(st + 128 + 8 * j);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = 16 * (e >> 1) + 2 * j + (e & 1);
      const float2 x = __ffma2_rn(__fadd2_rn(sv[idx], nm), c2, nl);
      const uint32_t bits = ((j < 4) ? w[e].x : w[e].y) >> (8 * (j & 3) + col0);
      const float2 pv = make_float2((bits & 1u) ? ex2(x.x) : 0.f, (bits & 2u) ? ex2(x.y) : 0.f);
      pr[idx] = pv;
      pk[idx] = pack16<BF16>(pv.x, pv.y);
    }
  }
}
// dS = (dP - delta) * P of the same elements, rounded once to 16 bits, unscaled.
template <bool BF16>
__device__ __forceinline__ void ds_frag(const float2* dp, const float2* pr, const float* st, uint32_t* dk) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 nd = *reinterpret_cast<const float2*>(st + 256 + 8 * j);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = 16 * (e >> 1) + 2 * j + (e & 1);
      const float2 d = __fmul2_rn(__fadd2_rn(dp[idx], nd), pr[idx]);
      dk[idx] = pack16<BF16>(d.x, d.y);
    }
  }
}

// The same for one query row of the dQ kernel, whose statistics are scalars. 32 columns (keys);
// MASKED: columns at or beyond `lim` (relative to this group's first column) get P = 0.
template <bool MASKED>
__device__ __forceinline__ void p_cols_by_key(const float2* sv, float2 nm, float2 c2, float2 nl, int lim, float2* pr) {
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    const float2 e = __ffma2_rn(__fadd2_rn(sv[x], nm), c2, nl);
    float2 q = make_float2(ex2(e.x), ex2(e.y));
    if constexpr (MASKED) {
      if (2 * x >= lim) q.x = 0.f;
      if (2 * x + 1 >= lim) q.y = 0.f;
    }
    pr[x] = q;
  }
}
// Under a boolean mask: bit x of `word` is the key of column x (32 columns).
__device__ __forceinline__ void p_cols_by_key_bits(const float2* sv, float2 nm, float2 c2, float2 nl, uint32_t word,
                                                   float2* pr) {
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    const float2 e = __ffma2_rn(__fadd2_rn(sv[x], nm), c2, nl);
    pr[x] = make_float2(((word >> (2 * x)) & 1u) ? ex2(e.x) : 0.f, ((word >> (2 * x + 1)) & 1u) ? ex2(e.y) : 0.f);
  }
}
template <bool BF16>
__device__ __forceinline__ void ds_cols_by_key(const float2* dp, const float2* pr, float2 nd, uint32_t* dk) {
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    const float2 d = __fmul2_rn(__fadd2_rn(dp[x], nd), pr[x]);
    dk[x] = pack16<BF16>(d.x, d.y);
  }
}

// ---------------------------------------------------------------------------------------
// dK / dV
// ---------------------------------------------------------------------------------------
template <int D, bool BF16, bool MASKW>
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
  constexpr int B_KV = 0;                 // 1       K, V landed
  constexpr int B_QREADY = 1;             // NSL     Q_i, dO_i, stats_i landed
  constexpr int B_QFREE = 1 + NSL;        // NSL     the MMAs that read the slot have retired
  constexpr int B_S = 1 + 2 * NSL;        // S^T(i) in TMEM
  constexpr int B_DP = 2 + 2 * NSL;       // dP^T(i) in TMEM
  constexpr int B_P = 3 + 2 * NSL;        // P^T(i) stored by both warpgroups (256 arrivals)
  constexpr int B_DS = 4 + 2 * NSL;       // dS^T(i) stored by both warpgroups
  constexpr int B_ACC = 5 + 2 * NSL;      // dV, dK complete
  constexpr int B_DRAIN = 6 + 2 * NSL;
  constexpr int B_PLO = 7 + 2 * NSL;      // the first 32 queries of P^T(i) stored by both warpgroups
  constexpr int N_BARS = 8 + 2 * NSL;
  static_assert(N_BARS * 8 + 16 <= 256, "barrier block too small");
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef KFA_TRACE
  const bool trace_on = (blockIdx.x == 0) && (lane == 0);
#endif

  // tile decode (groups of heads, tile-major inside); when causal the first key tiles see the most queries and come first
  int bh, kt;  // bh over batch x K / V heads
  decode_tile(blockIdx.x, p.B * p.Hkv, p.n_k128, bh, kt);
  const int b = bh / p.Hkv, hk = bh % p.Hkv;
  const int kv0 = kt * 128;  // relative to the sequence's first key
  int Sq = p.Sq, Skv = p.Skv, q_base = 0, k_base = 0, bc = b;  // bc: batch coordinate in the tensors
  if (p.cu_q != nullptr) {
    q_base = p.cu_q[b];
    Sq = p.cu_q[b + 1] - q_base;
    k_base = p.cu_k[b];
    Skv = p.cu_k[b + 1] - k_base;
    bc = 0;
    if (kv0 >= Skv) return;  // the whole CTA, before anything is set up
  }
  const int first_i = (p.P > 0) ? static_cast<int>((static_cast<long long>(kv0 / p.P) * p.P) / 128) : 0;
  // steps: for every query head of this K / V head's group, the query tiles that see these keys
  const int n_per = max((Sq + 127) / 128 - first_i, 0);
  int n_steps = n_per * p.group;
  const bool ragged_keys = kv0 + 128 > Skv;
  const int i_full = (p.P > 0 && !ragged_keys) ? first_full_tile(kv0, p.P) : 0;  // query tiles before it are masked steps
  // boolean masks with a tile table: the (query head, query tile) steps this CTA runs, in shared memory
  uint32_t* s_list = reinterpret_cast<uint32_t*>(smem + Cfg::KV_SMEM_TILES + 256);
  const bool use_list = MASKW && p.mt != nullptr;

  if (tid == 0) {
    mbar_init(bar(B_KV), 1);
    for (int i = 0; i < NSL; ++i) {
      mbar_init(bar(B_QREADY + i), 1);
      mbar_init(bar(B_QFREE + i), 1);
    }
    mbar_init(bar(B_S), 1);
    mbar_init(bar(B_DP), 1);
    mbar_init(bar(B_P), 256);
    mbar_init(bar(B_PLO), 256);
    mbar_init(bar(B_DS), 256);
    mbar_init(bar(B_ACC), 1);
    mbar_init(bar(B_DRAIN), 1);
    *s_abort = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(s_tmem), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if constexpr (MASKW) {
    if (use_list && warp == 1) {
      int count = 0;
      for (int g = 0; g < p.group; ++g) {
        const int* col = p.mt + bc * p.mt_sb + (hk * p.group + g) * p.mt_sh + kt;
        for (int i0 = 0; i0 < n_per; i0 += 32) {
          const int i = i0 + lane;
          const bool seen = i < n_per && __ldg(col + static_cast<long long>(i) * p.mt_row) != 0;
          const unsigned m = __ballot_sync(0xffffffffu, seen);
          if (seen) s_list[count + __popc(m & ((1u << lane) - 1u))] = (static_cast<uint32_t>(g) << 16) | static_cast<uint32_t>(i);
          count += __popc(m);
        }
      }
      if (lane == 0) s_tmem[2] = static_cast<uint32_t>(count);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  if (use_list) n_steps = static_cast<int>(s_tmem[2]);
  // step s -> query tile and query head
  auto tile_of = [&](int s) { return use_list ? static_cast<int>(s_list[s] & 0xffffu) : first_i + s % n_per; };
  auto head_of = [&](int s) { return hk * p.group + (use_list ? static_cast<int>(s_list[s] >> 16) : s / n_per); };
  const Ctl ctl{s_abort, p.status};
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
        tma_load_4d(sK + ch * Cfg::CHUNK_BYTES, &tmK, bar(B_KV), ch * Cfg::CHUNK_COLS, k_base + kv0, hk, bc);
        tma_load_4d(sV + ch * Cfg::CHUNK_BYTES, &tmV, bar(B_KV), ch * Cfg::CHUNK_COLS, k_base + kv0, hk, bc);
      }
      bool ok = true;
      int issued = 0;
      for (int s = 0; s < n_steps; ++s) {
        const int slot = s % NSL, use = s / NSL;
        if (use > 0) ok = mbar_wait(bar(B_QFREE + slot), (use - 1) & 1, ctl, 11);
        if (!ok) break;
        const int i = tile_of(s);
        const int head = head_of(s);
        const uint32_t base = sSlot + slot * Cfg::KV_SLOT_BYTES;
        mbar_expect_tx(bar(B_QREADY + slot), 2 * Cfg::TILE_BYTES + STATS_BYTES);
        for (int ch = 0; ch < CH; ++ch) {
          tma_load_4d(base + ch * Cfg::CHUNK_BYTES, &tmQ, bar(B_QREADY + slot), ch * Cfg::CHUNK_COLS, q_base + i * 128, head, bc);
          tma_load_4d(base + Cfg::TILE_BYTES + ch * Cfg::CHUNK_BYTES, &tmDO, bar(B_QREADY + slot), ch * Cfg::CHUNK_COLS,
                      q_base + i * 128, head, bc);
        }
        bulk_load(base + 2 * Cfg::TILE_BYTES,
                  p.stats + (static_cast<long long>(b) * p.H + head) * p.stats_sh + i * 384ll,
                  STATS_BYTES, bar(B_QREADY + slot));
        issued = s + 1;
      }
      if (!ok) {  // aborting: let the copies in flight land before the CTA gives up its shared memory
        mbar_drain(bar(B_KV), 0);
        for (int s = max(issued - NSL, 0); s < issued; ++s) mbar_drain(bar(B_QREADY + s % NSL), (s / NSL) & 1);
      }
    }
  } else if (warp == 8) {
    // =========================== MMA issue ===========================
    if (n_steps > 0) {
      const bool lead = elect_one();
      constexpr uint32_t IDESC_S = make_idesc(BF16, false, 128, 128);
      constexpr uint32_t IDESC_ACC = make_idesc(BF16, true, 128, D);
      const uint32_t tST = tmem + Cfg::TM_S, tDP = tmem + Cfg::TM_DP;
      const uint32_t tDV = tmem + Cfg::TM_ACC0, tDK = tmem + Cfg::TM_ACC1;
      const uint32_t k_lo = sdesc_lo(sK, 16), v_lo = sdesc_lo(sV, 16);
      bool ok = mbar_wait_warp(bar(B_KV), 0, ctl, 12);
      if (ok) ok = mbar_wait_warp(bar(B_QREADY + 0), 0, ctl, 13);
      if (ok) {
        tc_fence_after();
        issue_kmajor_n128<D>(lead, tST, k_lo, sdesc_lo(sSlot, 16), IDESC_S);
        umma_commit_lead(lead, bar(B_S));
        issue_kmajor_n128<D>(lead, tDP, v_lo, sdesc_lo(sSlot + Cfg::TILE_BYTES, 16), IDESC_S);
        umma_commit_lead(lead, bar(B_DP));
      }
      for (int s = 0; s < n_steps && ok; ++s) {
        const int slot = s % NSL;
        const uint32_t q_s = sSlot + slot * Cfg::KV_SLOT_BYTES;
        const uint32_t do_s = q_s + Cfg::TILE_BYTES;
        const int nslot = (s + 1) % NSL;
        const uint32_t q_n = sSlot + nslot * Cfg::KV_SLOT_BYTES;
        const uint32_t do_n = q_n + Cfg::TILE_BYTES;
        const bool more = s + 1 < n_steps;
        // dV += P^T(i) dO_i in two parts (the first 32 queries of each warpgroup's P^T are signalled
        // early, so the tensor core starts while the other exponentials are computed), then S^T(i+1)
        // may overwrite the P^T columns
        TR(3, s, 0, 0);
        ok = mbar_wait_warp(bar(B_PLO), s & 1, ctl, 14);
        if (!ok) break;
        TR(3, s, 0, 1);
        tc_fence_after();
        issue_tmemA_k64<D>(lead, tDV, tST, sdesc_lo(do_s, Cfg::CHUNK_BYTES), IDESC_ACC, s > 0, 0);
        ok = mbar_wait_warp(bar(B_P), s & 1, ctl, 20);
        if (!ok) break;
        TR(3, s, 0, 2);
        tc_fence_after();
        issue_tmemA_k64<D>(lead, tDV, tST, sdesc_lo(do_s, Cfg::CHUNK_BYTES), IDESC_ACC, s > 0, 1);
        if (more) {
          ok = mbar_wait_warp(bar(B_QREADY + nslot), ((s + 1) / NSL) & 1, ctl, 15);
          if (!ok) break;
          issue_kmajor_n128<D>(lead, tST, k_lo, sdesc_lo(q_n, 16), IDESC_S);
          umma_commit_lead(lead, bar(B_S));
        }
        TR(3, s, 0, 3);
        // dK += dS^T(i) Q_i, then dP^T(i+1) may overwrite the dS^T columns
        ok = mbar_wait_warp(bar(B_DS), s & 1, ctl, 16);
        if (!ok) break;
        TR(3, s, 0, 4);
        tc_fence_after();
        issue_tmemA_k128<D>(lead, tDK, tDP, sdesc_lo(q_s, Cfg::CHUNK_BYTES), IDESC_ACC, s > 0);
        umma_commit_lead(lead, bar(B_QFREE + slot));
        if (more) {
          issue_kmajor_n128<D>(lead, tDP, v_lo, sdesc_lo(do_n, 16), IDESC_S);
          umma_commit_lead(lead, bar(B_DP));
        }
        TR(3, s, 0, 5);
      }
      if (ok) umma_commit_lead(lead, bar(B_ACC));
      umma_commit_lead(lead, bar(B_DRAIN));
      mbar_drain(bar(B_DRAIN), 0);
    }
  } else {
    // =========================== P^T / dS^T and epilogue ===========================
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
    const float2 c2 = make_float2(p.c, p.c);
    bool ok = true;
    // boolean mask: for each of the thread's 4 key rows the two words of this warpgroup's 64 queries,
    // fetched a step ahead (rows past Skv read as hidden)
    const int* mkey[4] = {nullptr, nullptr, nullptr, nullptr};
    uint2 wnext[4];
    auto mask_fetch = [&](int s) {
      const int i = tile_of(s);
      const int head = head_of(s);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        wnext[e] = make_uint2(0u, 0u);
        if (mkey[e] != nullptr) wnext[e] = __ldg(reinterpret_cast<const uint2*>(mkey[e] + head * p.mwt_sh + 4 * i + 2 * hq));
      }
    };
    if constexpr (MASKW) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kr = kv0 + (warp & 3) * 32 + 16 * (e >> 1) + (lane >> 2) + 8 * (e & 1);
        if (kr < Skv) mkey[e] = p.mwt + bc * p.mwt_sb + static_cast<long long>(kr) * p.mwt_row;
      }
      if (n_steps > 0) mask_fetch(0);
    }
    StepWalk walk;
    for (int s = 0; s < n_steps; ++s, walk.next(n_per)) {
      uint2 wcur[4];
      if constexpr (MASKW) {
#pragma unroll
        for (int e = 0; e < 4; ++e) wcur[e] = wnext[e];
        if (s + 1 < n_steps) mask_fetch(s + 1);
      }
      const int slot = s % NSL;
      const int i = use_list ? tile_of(s) : first_i + walk.rel;
      const int q0 = i * 128 + 64 * hq + col0;  // query of this thread's first column
      // masked step: some (key, query) pair of this tile pair is hidden, or keys are padded
      const bool masked = ragged_keys || (p.P > 0 && i < i_full);
      if ((warp & 3) == 0) TR(hq, s, 0, 0);
      // (the step's statistics have landed too: S^T(i) was issued after the slot's copies had completed)
      ok = mbar_wait_warp(bar(B_S), s & 1, ctl, 18);
      if (!ok) break;
      if ((warp & 3) == 0) TR(hq, s, 0, 1);
      tc_fence_after();
      const float* st =
          reinterpret_cast<const float*>(smem + 2 * Cfg::TILE_BYTES + slot * Cfg::KV_SLOT_BYTES +
                                         2 * Cfg::TILE_BYTES) + 64 * hq + col0;
      float2 pr[32];  // fp32 P of this thread's 64 elements, kept for the dS phase
      // dP^T(i) is usually there already: tested now, settled after the exponentials
      const bool dp_probe = mbar_test(bar(B_DP), s & 1);
      {
        float2 sv[32];
        tmem_ld_16x256b_x8(tS, reinterpret_cast<uint32_t*>(sv));
        tmem_ld_16x256b_x8(tS + HALF, reinterpret_cast<uint32_t*>(sv + 16));
        tmem_wait_ld();
        if ((warp & 3) == 0) TR(hq, s, 0, 2);
        uint32_t pk[32];
        // 16-bit P^T goes over the first 32 of the 64 columns this warp has just read (all its lanes),
        // in two parts of 32 queries (16 packed columns) each
        if constexpr (MASKW)
          p_frag_bits<BF16, 0>(sv, st, c2, wcur, col0, pr, pk);
        else if (masked)
          p_frag<BF16, true, 0>(sv, st, c2, q0, qmin, pr, pk);
        else
          p_frag<BF16, false, 0>(sv, st, c2, q0, qmin, pr, pk);
        if ((warp & 3) == 0) TR(hq, s, 0, 7);
        tmem_st_16x128b_x4(tS, pk);
        tmem_st_16x128b_x4(tS + HALF, pk + 16);
        if constexpr (D > 64) {  // (at D <= 64 the dV MMA is too short for the early start to pay)
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(bar(B_PLO));
          if ((warp & 3) == 0) TR(hq, s, 0, 3);
        }
        if constexpr (MASKW)
          p_frag_bits<BF16, 4>(sv, st, c2, wcur, col0, pr, pk);
        else if (masked)
          p_frag<BF16, true, 4>(sv, st, c2, q0, qmin, pr, pk);
        else
          p_frag<BF16, false, 4>(sv, st, c2, q0, qmin, pr, pk);
        tmem_st_16x128b_x4(tS + 16, pk + 8);
        tmem_st_16x128b_x4(tS + HALF + 16, pk + 24);
      }
      tmem_wait_st();
      tc_fence_before();
      if constexpr (D <= 64) mbar_arrive(bar(B_PLO));
      mbar_arrive(bar(B_P));
      if ((warp & 3) == 0) TR(hq, s, 0, 4);
      ok = mbar_wait_warp_probed(dp_probe, bar(B_DP), s & 1, ctl, 19);
      if (!ok) break;
      if ((warp & 3) == 0) TR(hq, s, 0, 5);
      tc_fence_after();
      {
        float2 dp[32];
        tmem_ld_16x256b_x8(tDP, reinterpret_cast<uint32_t*>(dp));
        tmem_ld_16x256b_x8(tDP + HALF, reinterpret_cast<uint32_t*>(dp + 16));
        tmem_wait_ld();
        uint32_t dk[32];
        ds_frag<BF16>(dp, pr, st, dk);
        tmem_st_16x128b_x8(tDP, dk);
        tmem_st_16x128b_x8(tDP + HALF, dk + 16);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(B_DS));
      if ((warp & 3) == 0) TR(hq, s, 0, 6);
    }
    // ---- epilogue: warps 0-3 store dV, warps 4-7 store scale * dK ----
    const bool valid = key < Skv;
    const long long grow_row = static_cast<long long>(k_base) + key;
    uint8_t* grow;
    if (hq == 0)
      grow = reinterpret_cast<uint8_t*>(p.dv) + 2 * (bc * p.dv_sb + hk * p.dv_sh + grow_row * p.dv_ss);
    else
      grow = reinterpret_cast<uint8_t*>(p.dk) + 2 * (bc * p.dk_sb + hk * p.dk_sh + grow_row * p.dk_ss);
    float* grow32 = nullptr;
    if (p.acc_mode != 0)
      grow32 = (hq == 0 ? p.dv32 + (static_cast<long long>(b) * p.Hkv + hk) * p.dv32_sh
                        : p.dk32 + (static_cast<long long>(b) * p.Hkv + hk) * p.dk32_sh) +
               static_cast<long long>(key) * D;
    if (n_steps == 0) {
      if (valid && p.acc_mode == 0)
        for (int cc = 0; cc < D; cc += 8) *reinterpret_cast<uint4*>(grow + 2 * cc) = make_uint4(0, 0, 0, 0);
      if (valid && p.acc_mode == 1)
        for (int cc = 0; cc < D; cc += 4) *reinterpret_cast<float4*>(grow32 + cc) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      ok = mbar_wait_warp(bar(B_ACC), 0, ctl, 21) && ok;
      if (ok) {
        tc_fence_after();
        const uint32_t tacc = tmem + (hq ? Cfg::TM_ACC1 : Cfg::TM_ACC0) + lane_base;
        if (p.acc_mode == 0)
          store_acc_row<BF16, col_step(D)>(tacc, 0, D, hq ? p.scale : 1.0f, grow, valid);
        else
          store_acc_row_f32<col_step(D)>(tacc, 0, D, hq ? p.scale : 1.0f, grow32, valid, p.acc_mode == 2);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) {  // gave up (or an earlier kernel did): the rows of this CTA read as NaN
    const int r1 = min(kv0 + 128, Skv);
    if (p.acc_mode == 0) {
      fill_rows_nan16(reinterpret_cast<uint8_t*>(p.dk) + 2 * (bc * p.dk_sb + hk * p.dk_sh), p.dk_ss, k_base + kv0, k_base + r1, D);
      fill_rows_nan16(reinterpret_cast<uint8_t*>(p.dv) + 2 * (bc * p.dv_sb + hk * p.dv_sh), p.dv_ss, k_base + kv0, k_base + r1, D);
    } else if (r1 > kv0) {
      const long long bhl = static_cast<long long>(b) * p.Hkv + hk;
      fill_nan32(p.dk32 + bhl * p.dk32_sh + static_cast<long long>(kv0) * D, static_cast<long long>(r1 - kv0) * D);
      fill_nan32(p.dv32 + bhl * p.dv32_sh + static_cast<long long>(kv0) * D, static_cast<long long>(r1 - kv0) * D);
    }
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// dQ
// ---------------------------------------------------------------------------------------
template <int D, bool BF16, bool MASKW>
__global__ void __launch_bounds__(BWD_THREADS, 1)
kfa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                  const BwdParams p) {
  using Cfg = BwdCfg<D>;
  constexpr int CH = Cfg::CHUNKS;
  constexpr int NK = Cfg::NK, NV = Cfg::NV;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base;
  const uint32_t sDO = smem_base + Cfg::TILE_BYTES;
  const uint32_t sKr = smem_base + 2 * Cfg::TILE_BYTES;         // K ring
  const uint32_t sVr = smem_base + (2 + NK) * Cfg::TILE_BYTES;  // V ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::Q_SMEM_TILES);
  constexpr int B_Q = 0;                       // Q, dO landed
  constexpr int B_KREADY = 1;                  // NK
  constexpr int B_KFREE = 1 + NK;              // NK   dQ(j), the last reader of K_j, has retired
  constexpr int B_VREADY = 1 + 2 * NK;         // NV
  constexpr int B_VFREE = 1 + 2 * NK + NV;     // NV   dP(j), the only reader of V_j, has retired
  constexpr int B_S = 1 + 2 * NK + 2 * NV;     // S(j) in TMEM
  constexpr int B_DP = B_S + 1;                // dP(j) in TMEM
  constexpr int B_SREAD = B_S + 2;             // both warpgroups have read S(j) (256 arrivals)
  constexpr int B_DS = B_S + 3;                // dS(j) stored by both warpgroups
  constexpr int B_ACC = B_S + 4;
  constexpr int B_DRAIN = B_S + 5;
  constexpr int B_DPREAD = B_S + 6;            // both warpgroups hold dP(j) in registers (256 arrivals)
  constexpr int B_DSFREE = B_S + 7;            // 2: dQ(j), which read dS buffer j % 2, has retired
  constexpr int N_BARS = B_S + 9;
  static_assert(N_BARS * 8 + 16 <= 256, "barrier block too small");
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  int bh, t;
  decode_tile(blockIdx.x, p.B * p.H, p.n_q128, bh, t);
  const int qt = (p.P > 0) ? (p.n_q128 - 1 - t) : t;
  const int b = bh / p.H, h = bh % p.H;
  const int row0 = qt * 128;  // relative to the sequence's first row
  int Sq = p.Sq, Skv = p.Skv, q_base = 0, k_base = 0, bc = b;  // bc: batch coordinate in the tensors
  if (p.cu_q != nullptr) {
    q_base = p.cu_q[b];
    Sq = p.cu_q[b + 1] - q_base;
    k_base = p.cu_k[b];
    Skv = p.cu_k[b + 1] - k_base;
    bc = 0;
    if (row0 >= Sq || Skv <= 0) return;  // the whole CTA, before anything is set up
  }
  const int last = min(row0 + 127, Sq - 1);
  int n_steps = (key_limit(last, p.P, Skv) + 127) / 128;
  const int n_unmasked = key_limit(row0, p.P, Skv) / 128;
  // boolean masks with a tile table: the key tiles this CTA visits, in shared memory
  uint16_t* s_list = reinterpret_cast<uint16_t*>(smem + Cfg::Q_SMEM_TILES + 256);
  const bool use_list = MASKW && p.mt != nullptr;

  if (tid == 0) {
    mbar_init(bar(B_Q), 1);
    for (int i = 0; i < NK; ++i) {
      mbar_init(bar(B_KREADY + i), 1);
      mbar_init(bar(B_KFREE + i), 1);
    }
    for (int i = 0; i < NV; ++i) {
      mbar_init(bar(B_VREADY + i), 1);
      mbar_init(bar(B_VFREE + i), 1);
    }
    mbar_init(bar(B_S), 1);
    mbar_init(bar(B_DP), 1);
    mbar_init(bar(B_SREAD), 256);
    mbar_init(bar(B_DS), 256);
    mbar_init(bar(B_ACC), 1);
    mbar_init(bar(B_DRAIN), 1);
    mbar_init(bar(B_DPREAD), 256);
    mbar_init(bar(B_DSFREE + 0), 1);
    mbar_init(bar(B_DSFREE + 1), 1);
    *s_abort = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(s_tmem), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if constexpr (MASKW) {
    if (use_list && warp == 1) {
      const int* trow = p.mt + bc * p.mt_sb + h * p.mt_sh + static_cast<long long>(qt) * p.mt_row;
      int count = 0;
      for (int j0 = 0; j0 < n_steps; j0 += 32) {
        const int j = j0 + lane;
        const bool seen = j < n_steps && __ldg(trow + j) != 0;
        const unsigned m = __ballot_sync(0xffffffffu, seen);
        if (seen) s_list[count + __popc(m & ((1u << lane) - 1u))] = static_cast<uint16_t>(j);
        count += __popc(m);
      }
      if (count == 0) {  // nothing visible: one tile still runs, so that the rows get their zeros
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
  if (use_list) n_steps = static_cast<int>(s_tmem[2]);
  auto tile_of = [&](int it) { return use_list ? static_cast<int>(s_list[it]) : it; };
  const Ctl ctl{s_abort, p.status};
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
        tma_load_4d(sQ + ch * Cfg::CHUNK_BYTES, &tmQ, bar(B_Q), ch * Cfg::CHUNK_COLS, q_base + row0, h, bc);
        tma_load_4d(sDO + ch * Cfg::CHUNK_BYTES, &tmDO, bar(B_Q), ch * Cfg::CHUNK_COLS, q_base + row0, h, bc);
      }
      bool ok = true;
      int issued_k = 0, issued_v = 0;
      for (int j = 0; j < n_steps; ++j) {
        const int ks = j % NK, vs = j % NV;
        if (j >= NK) ok = mbar_wait(bar(B_KFREE + ks), (j / NK - 1) & 1, ctl, 51);
        if (!ok) break;
        mbar_expect_tx(bar(B_KREADY + ks), Cfg::TILE_BYTES);
        for (int ch = 0; ch < CH; ++ch)
          tma_load_4d(sKr + ks * Cfg::TILE_BYTES + ch * Cfg::CHUNK_BYTES, &tmK, bar(B_KREADY + ks), ch * Cfg::CHUNK_COLS,
                      k_base + tile_of(j) * 128, h / p.group, bc);
        issued_k = j + 1;
        if (j >= NV) ok = mbar_wait(bar(B_VFREE + vs), (j / NV - 1) & 1, ctl, 52);
        if (!ok) break;
        mbar_expect_tx(bar(B_VREADY + vs), Cfg::TILE_BYTES);
        for (int ch = 0; ch < CH; ++ch)
          tma_load_4d(sVr + vs * Cfg::TILE_BYTES + ch * Cfg::CHUNK_BYTES, &tmV, bar(B_VREADY + vs), ch * Cfg::CHUNK_COLS,
                      k_base + tile_of(j) * 128, h / p.group, bc);
        issued_v = j + 1;
      }
      if (!ok) {  // aborting: let the copies in flight land before the CTA gives up its shared memory
        mbar_drain(bar(B_Q), 0);
        for (int j = max(issued_k - NK, 0); j < issued_k; ++j) mbar_drain(bar(B_KREADY + j % NK), (j / NK) & 1);
        for (int j = max(issued_v - NV, 0); j < issued_v; ++j) mbar_drain(bar(B_VREADY + j % NV), (j / NV) & 1);
      }
    }
  } else if (warp == 8) {
    // MMA issue: the whole warp converged, one elected lane issues.
    {
      const bool lead = elect_one();
      constexpr uint32_t IDESC_S = make_idesc(BF16, false, 128, 128);
      constexpr uint32_t IDESC_ACC = make_idesc(BF16, true, 128, D);
      const uint32_t tS = tmem + Cfg::TM_S, tDP = tmem + Cfg::TM_DP, tDQ = tmem + Cfg::TM_ACC0;
      const uint32_t q_lo = sdesc_lo(sQ, 16), do_lo = sdesc_lo(sDO, 16);
      bool ok = mbar_wait_warp(bar(B_Q), 0, ctl, 53);
      if (ok) ok = mbar_wait_warp(bar(B_KREADY + 0), 0, ctl, 54);
      if (ok) {
        tc_fence_after();
        issue_kmajor_n128<D>(lead, tS, q_lo, sdesc_lo(sKr, 16), IDESC_S);
        umma_commit_lead(lead, bar(B_S));
        ok = mbar_wait_warp(bar(B_VREADY + 0), 0, ctl, 55);
      }
      if (ok) {
        tc_fence_after();
        issue_kmajor_n128<D>(lead, tDP, do_lo, sdesc_lo(sVr, 16), IDESC_S);
        umma_commit_lead(lead, bar(B_DP));
        umma_commit_lead(lead, bar(B_VFREE + 0));
      }
      for (int j = 0; j < n_steps && ok; ++j) {
        const uint32_t k_s = sKr + (j % NK) * Cfg::TILE_BYTES;
        const int nk = (j + 1) % NK, nv = (j + 1) % NV;
        const bool more = j + 1 < n_steps;
        if (more) {  // S(j+1) as soon as the warpgroups hold S(j) in registers
          ok = mbar_wait_warp(bar(B_KREADY + nk), ((j + 1) / NK) & 1, ctl, 56);
          if (ok) ok = mbar_wait_warp(bar(B_SREAD), j & 1, ctl, 57);
          if (!ok) break;
          tc_fence_after();
          issue_kmajor_n128<D>(lead, tS, q_lo, sdesc_lo(sKr + nk * Cfg::TILE_BYTES, 16), IDESC_S);
          umma_commit_lead(lead, bar(B_S));
        }
        auto issue_dP_next = [&]() {
          ok = mbar_wait_warp(bar(B_VREADY + nv), ((j + 1) / NV) & 1, ctl, 59);
          if (ok && Cfg::DS_OWN) ok = mbar_wait_warp(bar(B_DPREAD), j & 1, ctl, 63);
          if (!ok) return;
          tc_fence_after();
          issue_kmajor_n128<D>(lead, tDP, do_lo, sdesc_lo(sVr + nv * Cfg::TILE_BYTES, 16), IDESC_S);
          umma_commit_lead(lead, bar(B_DP));
          umma_commit_lead(lead, bar(B_VFREE + nv));
        };
        // own dS columns: dP(j+1) as soon as the warpgroups hold dP(j) in registers
        if (Cfg::DS_OWN && more) issue_dP_next();
        if (!ok) break;
        // dQ += dS(j) K_j
        ok = mbar_wait_warp(bar(B_DS), j & 1, ctl, 58);
        if (!ok) break;
        tc_fence_after();
        if constexpr (Cfg::DS_OWN) {
          issue_tmemA_k128_packed<D>(lead, tDQ, tmem + Cfg::TM_DS + 64 * (j & 1), sdesc_lo(k_s, Cfg::CHUNK_BYTES), IDESC_ACC, j > 0);
          umma_commit_lead(lead, bar(B_KFREE + j % NK));
          umma_commit_lead(lead, bar(B_DSFREE + (j & 1)));
        } else {
          issue_tmemA_k128<D>(lead, tDQ, tDP, sdesc_lo(k_s, Cfg::CHUNK_BYTES), IDESC_ACC, j > 0);
          umma_commit_lead(lead, bar(B_KFREE + j % NK));
        }
        // dS over the dP columns: dP(j+1) may overwrite them once dQ(j) is issued
        if (!Cfg::DS_OWN && more) issue_dP_next();
        if (!ok) break;
      }
      if (ok) umma_commit_lead(lead, bar(B_ACC));
      umma_commit_lead(lead, bar(B_DRAIN));
      mbar_drain(bar(B_DRAIN), 0);
    }
  } else {
    const int hk = warp >> 2;  // which 64 key columns of every tile
    const int r_in = tid & 127;
    const int row = row0 + r_in;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + Cfg::TM_S + 64 * hk + lane_base;
    const uint32_t tDP = tmem + Cfg::TM_DP + 64 * hk + lane_base;
    const uint32_t tDS = tmem + Cfg::TM_DS + 32 * hk + lane_base;  // this warpgroup's 32 packed columns of buffer 0
    const float* st = p.stats + static_cast<long long>(bh) * p.stats_sh + qt * 384ll;
    const float2 nm = make_float2(st[r_in], st[r_in]);                // -m
    const float2 nl = make_float2(st[128 + r_in], st[128 + r_in]);    // -log2 l
    const float2 nd = make_float2(st[256 + r_in], st[256 + r_in]);    // -delta
    const int my_limit = key_limit(min(row, Sq - 1), p.P, Skv);
    const float2 c2 = make_float2(p.c, p.c);
    bool ok = true;
    // boolean mask: the two words of this row for the warpgroup's 64 keys of a tile, fetched a tile ahead
    const uint2* mrow = nullptr;
    uint2 mnext = make_uint2(0u, 0u);
    if constexpr (MASKW) {
      mrow = reinterpret_cast<const uint2*>(p.mw + bc * p.mw_sb + h * p.mw_sh +
                                            static_cast<long long>(min(row, Sq - 1)) * p.mw_row + 2 * hk);
      if (n_steps > 0) mnext = __ldg(mrow + 2 * tile_of(0));
    }
    for (int j = 0; j < n_steps; ++j) {  // j counts visited tiles (tile_of(j) is the key tile)
      const uint2 mcur = mnext;
      if constexpr (MASKW) {
        if (j + 1 < n_steps) mnext = __ldg(mrow + 2 * tile_of(j + 1));
      }
      ok = mbar_wait_warp(bar(B_S), j & 1, ctl, 60);
      if (!ok) break;
      tc_fence_after();
      const int lim = my_limit - j * 128 - 64 * hk;  // visible columns of this warpgroup (masked tiles)
      float2 pr[32];
      bool dp_probe;
      {
        float2 sv[32];
        tmem_ld32(tS, reinterpret_cast<uint32_t*>(sv));
        tmem_ld32(tS + 32, reinterpret_cast<uint32_t*>(sv + 16));
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(bar(B_SREAD));  // S(j) is in registers: the tensor core may write S(j+1)
        dp_probe = mbar_test(bar(B_DP), j & 1);  // dP(j) is usually there already: settled after the exponentials
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          if constexpr (MASKW)
            p_cols_by_key_bits(sv + 16 * g, nm, c2, nl, g ? mcur.y : mcur.x, pr + 16 * g);
          else if (j >= n_unmasked)
            p_cols_by_key<true>(sv + 16 * g, nm, c2, nl, lim - 32 * g, pr + 16 * g);
          else
            p_cols_by_key<false>(sv + 16 * g, nm, c2, nl, 32, pr + 16 * g);
        }
      }
      ok = mbar_wait_warp_probed(dp_probe, bar(B_DP), j & 1, ctl, 61);
      if (!ok) break;
      tc_fence_after();
      {
        float2 dp[32];
        tmem_ld32(tDP, reinterpret_cast<uint32_t*>(dp));
        tmem_ld32(tDP + 32, reinterpret_cast<uint32_t*>(dp + 16));
        // own dS columns: the buffer of this step was last read by dQ(j-2), retired long ago: tested while the loads fly
        const bool free_probe = !Cfg::DS_OWN || (j < 2) || mbar_test(bar(B_DSFREE + (j & 1)), ((j >> 1) - 1) & 1);
        tmem_wait_ld();
        if constexpr (Cfg::DS_OWN) {
          tc_fence_before();
          mbar_arrive(bar(B_DPREAD));  // dP(j) is in registers: the tensor core may write dP(j+1)
          if (j >= 2) {
            ok = mbar_wait_warp_probed(free_probe, bar(B_DSFREE + (j & 1)), ((j >> 1) - 1) & 1, ctl, 64);
            if (!ok) break;
          }
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint32_t dk[16];
          ds_cols_by_key<BF16>(dp + 16 * g, pr + 16 * g, nd, dk);
          // 16-bit dS into its own columns, or over dP columns this thread has already read
          tmem_st16(Cfg::DS_OWN ? tDS + 64 * (j & 1) + 16 * g : tDP + 16 * g, dk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(B_DS));
    }
    ok = mbar_wait_warp(bar(B_ACC), 0, ctl, 62) && ok;
    if (ok) {
      tc_fence_after();
      // the two warpgroups share the row's D columns, split at a multiple of 16
      constexpr int SPLIT = ((D / 2 + 15) / 16) * 16;
      constexpr int W = (SPLIT % 32 == 0 && (D - SPLIT) % 32 == 0) ? 32 : 16;
      const int c0 = hk ? SPLIT : 0, nc = hk ? D - SPLIT : SPLIT;
      if (p.acc_mode == 0) {
        uint8_t* grow = reinterpret_cast<uint8_t*>(p.dq) +
                        2 * (bc * p.dq_sb + h * p.dq_sh + static_cast<long long>(q_base + row) * p.dq_ss);
        store_acc_row<BF16, W>(tmem + Cfg::TM_ACC0 + lane_base, c0, nc, p.scale, grow, row < Sq);
      } else {
        float* grow32 = p.dq32 + (static_cast<long long>(b) * p.H + h) * p.dq32_sh + static_cast<long long>(row) * D;
        store_acc_row_f32<W>(tmem + Cfg::TM_ACC0 + lane_base, c0, nc, p.scale, grow32, row < Sq, p.acc_mode == 2);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) {  // gave up (or an earlier kernel did): the rows of this CTA read as NaN
    const int r1 = min(row0 + 128, Sq);
    if (p.acc_mode == 0)
      fill_rows_nan16(reinterpret_cast<uint8_t*>(p.dq) + 2 * (bc * p.dq_sb + h * p.dq_sh), p.dq_ss, q_base + row0, q_base + r1, D);
    else if (r1 > row0)
      fill_nan32(p.dq32 + (static_cast<long long>(b) * p.H + h) * p.dq32_sh + static_cast<long long>(row0) * D,
                 static_cast<long long>(r1 - row0) * D);
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

}  // namespace kfa
