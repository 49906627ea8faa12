// Thin inline-PTX wrappers for the sm_100a features the attention kernels use:
// mbarriers with bounded waits, TMA tile loads, tensor-memory (TMEM) allocation,
// tcgen05 MMAs with shared-memory / TMEM operands, TMEM loads and stores.
//
// Every wait in this file is bounded: a wait that runs out sets the CTA's abort flag and
// a status word in global memory, and returns false; the caller leaves its loop and
// falls through to the kernel's common teardown, which frees TMEM. No kernel here can
// spin forever.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace kfa {

// Status codes written to the device status word (first failure wins).
enum : int {
  KFA_DEV_OK = 0,
  // 100 + id of the wait that gave up; every wait in the library has an id of its own:
  // 1-9 forward, 11-21 dK/dV kernel, 30-50 fused backward, 51-62 dQ kernel, 91-99 self-test and diagnostics
  KFA_DEV_TIMEOUT_BASE = 100,
  KFA_DEV_BAD_SMEM_BASE = 99,  // the dynamic shared memory of a kernel that needs it did not start on a 1 KB boundary
};

// Longest time a wait may take, in SM clock cycles: ~2 s at 1.9 GHz. Legitimate waits last
// microseconds; the margin is for a CTA that is preempted or time-sliced (the cycle counter keeps
// running) or replayed under a profiler.
#ifndef KFA_WAIT_CYCLES
#define KFA_WAIT_CYCLES 4000000000ll
#endif
// The limit of the waits of the teardown itself (a CTA that gives up still lets the MMAs it has issued
// retire and the copies it has started land before it frees its tensor memory and shared memory):
// never shortened, also not in the test build that sets a tiny KFA_WAIT_CYCLES.
#define KFA_DRAIN_CYCLES 4000000000ll

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Make generic-proxy writes to shared memory visible to the async proxy (TMA, MMA).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// A limit this short only occurs in the test build whose waits are meant to run out: it then polls
// without letting the hardware suspend the thread, and looks at the clock on every turn.
constexpr bool KFA_SHORT_WAITS = (KFA_WAIT_CYCLES < 1000000ll);

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  if constexpr (KFA_SHORT_WAITS) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return ok != 0;
}

// Non-blocking test of a phase (try_wait may suspend the thread for a while when the phase is incomplete;
// this never does): for the early tests of mbar_wait_warp_probed.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Per-CTA control block: abort flag in shared memory, status word in global memory.
struct Ctl {
  volatile int* s_abort;
  int* g_status;
};

// Bounded wait for the phase with the given parity to complete. Returns false when the
// CTA is aborting (this wait or another ran out of time, or another CTA reported a failure).
// The first test stands apart from the polling loop: a wait whose phase has already completed (most of them,
// in a pipeline that runs ahead) costs one try_wait and, for a warp, one vote.
__device__ __forceinline__ bool mbar_wait_poll(uint32_t bar, uint32_t parity, volatile int* s_abort, int* g_status,
                                            int site) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (KFA_SHORT_WAITS || (++spins & 31u) == 0u) {
      if (*s_abort) return false;
      if ((spins & 1023u) == 0u && *reinterpret_cast<volatile int*>(g_status) != 0) {
        *s_abort = 1;
        return false;
      }
      if (clock64() - t0 > KFA_WAIT_CYCLES) {
        *s_abort = 1;
        atomicCAS(g_status, 0, KFA_DEV_TIMEOUT_BASE + site);
        return false;
      }
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const Ctl& ctl, int site) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_poll(bar, parity, ctl.s_abort, ctl.g_status, site);
}

// For a thread that gives up while copies it has started may still be in flight: waits (bounded, without
// touching the abort state) until the phase has completed, so that nothing lands in shared memory after
// the CTA has released it.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity) && clock64() - t0 < KFA_DRAIN_CYCLES) {
  }
}

// The same for a full warp about to run warp-aligned tcgen05 instructions: the warp reconverges
// and every lane gets the same answer (false if any lane gave up).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const Ctl& ctl, int site) {
  bool ok = mbar_try_wait(bar, parity);
  if (__all_sync(0xffffffffu, ok)) return true;  // the phase had completed: about 25 clk
  if (!ok) ok = mbar_wait_poll(bar, parity, ctl.s_abort, ctl.g_status, site);
  return __all_sync(0xffffffffu, ok);
}

// A test costs the thread its round trip to the barrier, about 50 clk, even when the phase completed long
// ago. Where the phase is usually complete well before it is needed, a warp tests it EARLY (`probed =
// mbar_test(...)`, issued ahead of independent work) and settles here when it needs the data: the
// round trip is hidden, and the data was complete when the early test saw it.
__device__ __forceinline__ bool mbar_wait_warp_probed(bool probed, uint32_t bar, uint32_t parity, const Ctl& ctl,
                                                      int site) {
  if (__all_sync(0xffffffffu, probed)) return true;
  return mbar_wait_warp(bar, parity, ctl, site);
}

// ----------------------------------------------------------------------------------
// TMA (tiled tensor loads, plain bulk loads), each into this CTA's own shared memory only.
// ----------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ----------------------------------------------------------------------------------
// Tensor memory
// ----------------------------------------------------------------------------------
// One full warp; ncols a power of two in 32..512. The base address lands in *smem_dst.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------------
// MMA descriptors
// ----------------------------------------------------------------------------------
// Instruction descriptor for kind::f16 (fp16 or bf16 operands, fp32 accumulate).
// bits [4,6) D format (1 = f32); [7,10) A format, [10,13) B format (0 = f16, 1 = bf16);
// bit 15 A major, bit 16 B major (0 = K-major, 1 = MN-major); [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, bool b_mn_major, int m, int n) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle. Addresses and offsets in bytes.
// bits [0,14) start >> 4; [16,30) leading byte offset >> 4; [32,46) stride byte offset >> 4;
// bits [46,48) = 1 (descriptor version of this architecture); [61,64) = 2 (128-byte swizzle).
//  K-major tile (rows of 64 16-bit elements = 128 B, as a 128B-swizzled TMA box writes them):
//    stride offset = 1024 (eight rows); leading offset unused.
//  MN-major tile (rows are K, 64 contiguous MN elements per row): stride offset = 1024 (eight
//    K rows); leading offset = distance between consecutive 64-element MN blocks.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) |
         (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; A holds 16-bit elements, two K values per 32-bit column.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---- the same, for an MMA warp that runs converged with one elected lane issuing ----
// The whole warp executes the role's control flow (so descriptor arithmetic stays warp-uniform and
// cheap); only the tcgen05 instruction itself is predicated on the elected lane. Descriptors are
// handled as 32-bit halves: the high word is the same for every tile of these kernels (stride
// offset 1024, descriptor version 1, 128-byte swizzle); advancing along K only adds to the low word
// (the address field cannot carry: shared memory addresses >> 4 fit in its 14 bits).
constexpr uint32_t SDESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);

// Head dims are handled as chunks of C columns, C the widest of 64, 32, 16 that divides the head dim: one TMA
// box of 128 rows x C columns per chunk, written with the swizzle whose span is the box's row (128, 64 or 32
// bytes), so that a tile of any head dim that is a multiple of 16 is loaded and multiplied without padding
// (the reference's chunking: src/kohakufa/sm100/config.py:15, 76-80).
__host__ __device__ constexpr int chunk_cols(int D) { return D % 64 == 0 ? 64 : (D % 32 == 0 ? 32 : 16); }
__host__ __device__ constexpr int chunk_bytes(int D) { return 128 * chunk_cols(D) * 2; }
// High descriptor word for a tile of such chunks: stride offset = eight rows of 2 C bytes; swizzle field
// 2 / 4 / 6 = 128 / 64 / 32 bytes. (K-major: the leading offset is unused. MN-major: rows are K, C contiguous
// MN elements per row, leading offset = distance between chunks.)
__host__ __device__ constexpr uint32_t sdesc_hi_for(int D) {
  return (static_cast<uint32_t>(16 * chunk_cols(D)) >> 4) | (1u << 14) |
         ((chunk_cols(D) == 64 ? 2u : (chunk_cols(D) == 32 ? 4u : 6u)) << 29);
}
// Byte offset of k-step kk (16 contraction elements) of a K-major tile made of such chunks.
__host__ __device__ constexpr uint32_t kstep_bytes(int D, int kk) {
  return static_cast<uint32_t>((kk / (chunk_cols(D) / 16)) * chunk_bytes(D) + (kk % (chunk_cols(D) / 16)) * 32);
}
// Byte offset of k-step kk (16 rows) of an MN-major tile made of such chunks.
__host__ __device__ constexpr uint32_t kstep_rows_bytes(int D, int kk) {
  return static_cast<uint32_t>(kk * 16 * chunk_cols(D) * 2);
}
// Columns of an fp32 accumulator moved per tensor-memory access in the row loops: 32, or 16 where the head
// dim is an odd multiple of 16.
__host__ __device__ constexpr int col_step(int D) { return D % 32 == 0 ? 32 : 16; }

__device__ __forceinline__ uint32_t sdesc_lo(uint32_t saddr, uint32_t lbo) {
  return ((saddr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16);
}

// True in exactly one lane of the (fully active) warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void umma_ss_lead(bool lead, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                             uint32_t idesc, uint32_t accumulate, uint32_t hi = SDESC_HI) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %6, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(hi),
      "r"(static_cast<uint32_t>(lead))
      : "memory");
}

__device__ __forceinline__ void umma_ts_lead(bool lead, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                             uint32_t idesc, uint32_t accumulate, uint32_t hi = SDESC_HI) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %6, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(hi),
      "r"(static_cast<uint32_t>(lead))
      : "memory");
}

__device__ __forceinline__ void umma_commit_lead(bool lead, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar), "r"(static_cast<uint32_t>(lead))
      : "memory");
}

// mbarrier arrives once every MMA this thread issued so far has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ----------------------------------------------------------------------------------
// TMEM <-> registers. Shape 32x32b: thread t of the warp owns lane (lane_base + t); register i
// is column (col + i). A warp may only touch lanes 32 * (warp_id % 4) .. + 31.
// ----------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
      "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Fragment shapes (16 TMEM lanes per instruction; a warp reaches its 32 lanes with lane offsets 0 and 16).
// Register <-> element maps, checked on hardware against the 32x32b shape:
//   ld.16x256b.x8 (16 lanes x 64 columns, 32 registers): thread l holds for column block j = 0..7
//     r[4j], r[4j+1] = (lane l/4, columns 8j + 2(l%4), +1);  r[4j+2], r[4j+3] = (lane l/4 + 8, same columns)
//   st.16x128b.x8 (16 lanes x 32 columns, 16 registers): r[2j] -> (lane l/4, column 4j + l%4),
//     r[2j+1] -> (lane l/4 + 8, same column)
// so a thread that packs the two adjacent fp32 columns it loaded into one 32-bit word of two 16-bit values
// stores exactly the word the 16-bit MMA operand layout wants at that lane.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// st.16x128b.x4: 16 lanes x 16 columns, 8 registers, same element map as the x8 form.
__device__ __forceinline__ void tmem_st_16x128b_x4(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x4.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}

// Sets the calling warpgroup's registers per thread (all four warps must call it). The kernel starts
// with LAUNCH per thread (what its thread count leaves of the 64 K registers, in eights): a budget above
// that waits until other warpgroups have released enough.
template <int N, int LAUNCH = 128>
__device__ __forceinline__ void reg_budget() {
  static_assert(N % 8 == 0 && N >= 24 && N <= 256, "register budget");
  if constexpr (N > LAUNCH) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
  } else if constexpr (N < LAUNCH) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
  }
}

// ----------------------------------------------------------------------------------
// What a CTA that gives up leaves behind: NaN in every output row it owns, so that a timed-out wait
// cannot pass for a result (0x7fff is a NaN in fp16 and in bf16). Called by all threads of the CTA.
// ----------------------------------------------------------------------------------
__device__ __forceinline__ void fill_rows_nan16(void* base, long long row_stride, int r0, int r1, int dim) {
  const int chunks = dim / 8;
  const uint4 nan8 = make_uint4(0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu);
  for (int i = threadIdx.x; i < (r1 - r0) * chunks; i += blockDim.x) {
    const long long r = r0 + i / chunks;
    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(base) + 2 * (r * row_stride + (i % chunks) * 8)) = nan8;
  }
}
__device__ __forceinline__ void fill_nan32(float* base, long long count) {
  for (long long i = threadIdx.x; i < count; i += blockDim.x) base[i] = __int_as_float(0x7fc00000);
}

template <int W>
__device__ __forceinline__ void tmem_ldw(uint32_t taddr, uint32_t* r) {
  if constexpr (W == 32) tmem_ld32(taddr, r);
  else tmem_ld16(taddr, r);
}
template <int W>
__device__ __forceinline__ void tmem_stw(uint32_t taddr, const uint32_t* r) {
  if constexpr (W == 32) tmem_st32(taddr, r);
  else tmem_st16(taddr, r);
}

// ----------------------------------------------------------------------------------
// Arithmetic helpers
// ----------------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two fp32 -> one 32-bit word of two 16-bit values (lo in the low half), round to nearest even.
template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// The fp32 values of the two 16-bit halves of a packed word.
template <bool BF16>
__device__ __forceinline__ float2 unpack16(uint32_t w) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
  }
}

template <bool BF16>
__device__ __forceinline__ float load16(const void* p) {
  if constexpr (BF16) {
    return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
  } else {
    return __half2float(*reinterpret_cast<const __half*>(p));
  }
}

}  // namespace kfa
