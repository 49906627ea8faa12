/*
 * kfa.h - C ABI of libkfa.so: flash-attention forward and backward for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a host binds instead of the reference's Triton launchers
 * (KohakuFA: src/kohakufa/sm100/fwd.py:1188-1232 attention_forward,
 *            src/kohakufa/sm100/bwd.py:1413-1482 attention_backward).
 *
 * Conventions
 *   - Every tensor is a [B, H, S, D] view described by KfaTensor4: element strides, last
 *     dimension contiguous, every other stride a multiple of 8 elements (16 bytes), base
 *     pointer 16-byte aligned (the reference's rule, src/kohakufa/sm100/op.py:53-55).
 *   - 16-bit data is fp16 (KFA_F16) or bf16 (KFA_BF16). D is a multiple of 16 up to 128 (the fused backward: 64 or 128). H of q is a multiple of
 *     H of k / v (grouped-query attention: query head h uses K / V head h / (H / Hkv)).
 *   - block = 0: dense. block = P > 0: key c is visible to query r iff c / P <= r / P
 *     (top-left aligned; P = 1 is token-causal) (tests/reference.py:6-12).
 *   - Calls enqueue work on `stream` (a cudaStream_t) of the CURRENT device and return without
 *     synchronising. They allocate no device memory: outputs and scratch are the caller's.
 *   - Return value: 0 on success, a negative KFA_ERR_* otherwise; kfa_last_error() then gives a
 *     message (thread-local).
 *   - `dev_status` points to one int32 in device memory, zero before the first call. A kernel
 *     whose internal wait ran out of time writes a nonzero code there and finishes early
 *     instead of hanging; later launches that see a nonzero word do nothing. The host reads
 *     it whenever it wants to (tests do after every call).
 */
#ifndef KFA_H_
#define KFA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KFA_ABI_VERSION 1

#define KFA_F16 0
#define KFA_BF16 1

#define KFA_OK 0
#define KFA_ERR_ARG (-1)      /* shape / stride / alignment / dtype not supported */
#define KFA_ERR_CUDA (-2)     /* a CUDA runtime or driver call failed */
#define KFA_ERR_SELFTEST (-3) /* kfa_selftest: results differ from the host computation */

typedef struct KfaTensor4 {
  void* ptr;
  int64_t shape[4];  /* B, H, S, D */
  int64_t stride[4]; /* in elements */
} KfaTensor4;

int kfa_abi_version(void);
const char* kfa_last_error(void);

/* Bytes of the backward's per-row statistics scratch for (B, H, Sq): fp32
 * [B*H, ceil(Sq/128), 3, 128] holding (m, log2 l, delta) per query row. */
int64_t kfa_bwd_stats_bytes(int64_t B, int64_t H, int64_t Sq);

/* Forward. out: [B, H, Sq, D]; lse: fp32 [B, H, 2, Sq] contiguous, plane 0 = row max m of the raw
 * (unscaled) scores, plane 1 = log2(l), l = sum exp2((S - m) * scale * log2 e).
 * Replaces attention_forward (fwd.py:1188-1232) + attention_fwd_kernel (fwd.py:1065-1136). */
int kfa_fwd(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
            float* lse, float scale, int block, int dtype, int* dev_status, void* stream);

/* Backward, step 1: delta = rowsum(dout * out) and the packed per-tile statistics.
 * Replaces _prepare_kernel (bwd.py:1358-1388). */
int kfa_bwd_prepare(const KfaTensor4* out, const KfaTensor4* dout, const float* lse, float* stats,
                    int dtype, void* stream);

/* Backward, step 2: dK and dV. Replaces the dK / dV half of attention_bwd_kernel (bwd.py:1248-1350). */
int kfa_bwd_dkdv(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
                 const float* stats, const KfaTensor4* dk, const KfaTensor4* dv, float scale, int block,
                 int dtype, int* dev_status, void* stream);

/* Backward, step 3: dQ. Replaces the dQ half of attention_bwd_kernel and _dq_convert_kernel
 * (bwd.py:1135-1232, 1391-1410). */
int kfa_bwd_dq(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
               const float* stats, const KfaTensor4* dq, float scale, int block, int dtype,
               int* dev_status, void* stream);

/* Backward, all three steps in stream order. Replaces attention_backward (bwd.py:1413-1482).
 * `stats` is scratch of kfa_bwd_stats_bytes(B, H, Sq) bytes. */
int kfa_bwd(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
            const KfaTensor4* dout, const float* lse, float* stats, const KfaTensor4* dq,
            const KfaTensor4* dk, const KfaTensor4* dv, float scale, int block, int dtype,
            int* dev_status, void* stream);

/* Backward as ONE main kernel (dK, dV and dQ from one P and one dS per tile pair, five matrix products
 * instead of the seven of kfa_bwd), the way the reference's backward works: replaces
 * attention_backward (bwd.py:1413-1482) with its fp32 dQ accumulator (bwd.py:1135-1232 reduce partition,
 * 1391-1410 _dq_convert_kernel). Three launches in stream order: statistics + zero-fill of the
 * accumulator, the fused kernel (dQ tiles are added to the accumulator with fp32 reduce-adds), conversion
 * of the accumulator to 16-bit dq. dK and dV are bit-identical to kfa_bwd's; dQ is identical up to the
 * order of its fp32 additions, which varies from run to run (use kfa_bwd where bit-reproducible
 * gradients are required).
 * `stats`: kfa_bwd_stats_bytes(B, H, Sq) bytes; `dq_acc`: kfa_bwd_dq_acc_bytes(B, H, Sq, D) bytes
 * (fp32, whole 128-row tiles: 4 * D bytes per padded query row), 16-byte aligned; both are scratch. */
int64_t kfa_bwd_dq_acc_bytes(int64_t B, int64_t H, int64_t Sq, int64_t D);
/* Its three launches one by one (kfa_bwd_fused = these in this order):
 *   kfa_bwd_prepare_fused  statistics as kfa_bwd_prepare, and zero-fills dq_acc   (bwd.py:1358-1388)
 *   kfa_bwd_fused_main     dK, dV written; dQ tiles added to dq_acc                 (bwd.py:1248-1350)
 *   kfa_bwd_dq_convert     dq = 16-bit(scale * dq_acc)                              (bwd.py:1391-1410) */
int kfa_bwd_prepare_fused(const KfaTensor4* out, const KfaTensor4* dout, const float* lse, float* stats,
                          float* dq_acc, int dtype, void* stream);
int kfa_bwd_fused_main(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
                       const float* stats, float* dq_acc, const KfaTensor4* dk, const KfaTensor4* dv,
                       float scale, int block, int dtype, int* dev_status, void* stream);
int kfa_bwd_dq_convert(const float* dq_acc, const KfaTensor4* dq, float scale, int dtype,
                       const int* dev_status, void* stream);
int kfa_bwd_fused(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
                  const KfaTensor4* dout, const float* lse, float* stats, float* dq_acc, const KfaTensor4* dq,
                  const KfaTensor4* dk, const KfaTensor4* dv, float scale, int block, int dtype,
                  int* dev_status, void* stream);

/* Packed variable-length batches. Replace attention_forward_varlen (fwd.py:1277-1320) and
 * attention_backward_varlen (bwd.py:1591-1647); the reference's host-built tile tables (fwd.py:1265-1274,
 * bwd.py:1559-1588) are not needed: the kernels read the sequence boundaries themselves.
 *
 * q / out / dout / dq are [1, H, Tq, D] views and k / v / dk / dv [1, Hkv, Tk, D] views of the packed
 * [T, H, D] tensors; sequence b (0 <= b < n_seqs) owns query rows cu_seqlens_q[b] .. cu_seqlens_q[b + 1]
 * and key rows cu_seqlens_k[b] .. cu_seqlens_k[b + 1] (int32[n_seqs + 1] in DEVICE memory, ascending,
 * first entry 0) and is its own attention problem: `block` applies inside each sequence. max_q / max_k:
 * the longest sequence's queries / keys (host ints: they size the grids, so no call reads device
 * memory on the host). lse is [1, H, 2, Tq]. `stats`: kfa_bwd_stats_bytes(n_seqs, H, max_q) bytes.
 * A sequence with queries but no keys is skipped (its output rows are left unwritten); rows of
 * neighbouring sequences that share a tile are read and masked, so they must hold finite numbers. */
int kfa_fwd_varlen(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
                   float* lse, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int n_seqs,
                   int max_q, int max_k, float scale, int block, int dtype, int* dev_status, void* stream);
int kfa_bwd_varlen(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
                   const KfaTensor4* dout, const float* lse, float* stats, const KfaTensor4* dq,
                   const KfaTensor4* dk, const KfaTensor4* dv, const int32_t* cu_seqlens_q,
                   const int32_t* cu_seqlens_k, int n_seqs, int max_q, int max_k, float scale, int block,
                   int dtype, int* dev_status, void* stream);

/* Boolean masks. Replace the mask arguments of attention_forward / attention_backward (fwd.py:1188-1232,
 * bwd.py:1413-1482: mask_words, mask_words_t) and the packing kernel (mask.py:32-72).
 *
 * A mask is passed as packed words, bit set = the key is visible: `words` hold 32 keys per 32-bit word
 * along each query row (bit c % 32 of word c / 32 is key c), `words_t` 32 queries per word along each key
 * row. Rows are 4 * ceil(n / 128) words long (whole 128-wide tiles) with zero bits past the end. The words
 * of row r of (batch b, head h) start at words + b * stride_batch + h * stride_head + r * stride_row
 * (in words; multiples of 4; a batch / head stride of 0 broadcasts one mask). A query row with no
 * visible key gets output 0 and zero gradients (its statistics are m = +inf, log2 l = 0).
 *
 * Optional tile table (replaces the reference's tile lists, mask.py:74-122): one int32 per (128 queries x
 * 128 keys) tile, nonzero = the tile holds a visible pair; tile (qt, kt) of (b, h) at any + b * stride_batch
 * + h * stride_head + qt * ceil(Skv / 128) + kt. With it the kernels skip tile pairs in which nothing is
 * visible (each CTA lists the tiles it visits in shared memory; where a list would not fit — more than
 * 1024 key tiles per row, 768 for the dQ kernel at D = 128, 2048 (query head, query tile) steps per key
 * tile — every tile is visited). NULL: every tile is visited. */
typedef struct KfaMaskWords {
  const int32_t* words;
  int64_t stride_batch, stride_head, stride_row;
} KfaMaskWords;
typedef struct KfaMaskTiles {
  const int32_t* any;
  int64_t stride_batch, stride_head;
} KfaMaskTiles;

/* mask: bytes, nonzero = visible, element (b, h, r, c) at mask[b * s[0] + h * s[1] + r * s[2] + c * s[3]]
 * with mask_batch x mask_heads x Sq x Skv elements. words: int32[mask_batch * mask_heads * Sq *
 * 4 ceil(Skv / 128)], words_t: int32[mask_batch * mask_heads * Skv * 4 ceil(Sq / 128)], both contiguous.
 * tiles (optional): int32[mask_batch * mask_heads * ceil(Sq / 128) * ceil(Skv / 128)], ZEROED by the
 * caller; the kernel sets the entries of tiles that hold a visible pair. */
int kfa_pack_mask(const void* mask, const int64_t* mask_stride, int mask_batch, int mask_heads, int Sq,
                  int Skv, int32_t* words, int32_t* words_t, int32_t* tiles, void* stream);
int kfa_fwd_masked(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
                   float* lse, const KfaMaskWords* words, const KfaMaskTiles* tiles, float scale, int dtype,
                   int* dev_status, void* stream);
int kfa_bwd_masked(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
                   const KfaTensor4* dout, const float* lse, float* stats, const KfaTensor4* dq,
                   const KfaTensor4* dk, const KfaTensor4* dv, const KfaMaskWords* words,
                   const KfaMaskWords* words_t, const KfaMaskTiles* tiles, float scale, int dtype,
                   int* dev_status, void* stream);

/* Backward without a scratch buffer from the caller. No counterpart in the reference (there the
 * launcher allocates its scratch from torch's caching allocator, bwd.py:1434-1439).
 *
 * kfa_bwd needs `stats`, scratch the caller has to allocate. Some hosts have no way to do that at the
 * point of the call: a binding from a runtime that owns no device allocator and only passes on the
 * tensors it was given, a serving loop that may not touch cudaMalloc because it synchronises the
 * device, a process whose memory is fully pre-carved. For them the library keeps ONE statistics
 * buffer of KFA_STATIC_SCRATCH_BYTES inside its own device image (every GPU that loads libkfa.so
 * holds these bytes until the process exits) and this entry point runs the same three kernels on it.
 * It calls no cudaMalloc, cudaFree or other allocating routine.
 *
 *   - Limit: kfa_bwd_stats_bytes(B, H, Sq) <= KFA_STATIC_SCRATCH_BYTES, i.e. B * H * ceil(Sq / 128) <=
 *     5461 query tiles (about 699,000 query rows). Larger problems are refused with KFA_ERR_ARG.
 *   - The first call on each device looks the buffer's device address up (one runtime query, with that
 *     device current). Make that first call outside any stream capture.
 *   - All calls on a device share the one buffer, which keeps the previous call's contents; each call
 *     rewrites every entry it reads, so nothing has to be cleared. Two calls whose kernels overlap on
 *     the GPU (different streams) race on it: serialise them, or use kfa_bwd with separate buffers. */
#define KFA_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int kfa_bwd_static_scratch(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v,
                           const KfaTensor4* out, const KfaTensor4* dout, const float* lse,
                           const KfaTensor4* dq, const KfaTensor4* dk, const KfaTensor4* dv, float scale,
                           int block, int dtype, int* dev_status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Context-parallel building blocks: one attention problem whose sequence is spread over several
 * GPUs, computed as (local queries) x (visiting keys / values) steps. Everything that crosses steps
 * stays in fp32: the unnormalised O with its (m, l) per row in the forward, dQ / dK / dV accumulators
 * in the backward; each is rounded to 16 bits once, by a finalize call. No counterpart in the
 * reference, which is single-GPU. The host side (who sends what to whom) is kohakufa_b200/ring.py.
 * --------------------------------------------------------------------------------------------- */

/* fp32 rows of D elements: row r of (b, h) starts at ptr + (b * H + h) * head_stride + r * D. */
typedef struct KfaAcc32 {
  float* ptr;
  int64_t head_stride; /* in floats */
} KfaAcc32;

/* One forward step: attention of q against the visiting k / v (block as in kfa_fwd). The partial
 * result is written to (merge = 0) or merged into (merge = 1) the carry: o_acc, and ml with m at
 * ml[(b*H+h) * ml_head_stride + r] and l at the same + ml_plane_stride. */
int kfa_cp_fwd_step(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaAcc32* o_acc,
                    float* ml, int64_t ml_head_stride, int64_t ml_plane_stride, int merge, float scale,
                    int block, int dtype, int* dev_status, void* stream);

/* out = o_acc / l rounded to 16 bits; lse [B, H, 2, Sq] = (m, log2 l), as kfa_fwd would have left them. */
int kfa_cp_fwd_finalize(const KfaAcc32* o_acc, const float* ml, int64_t ml_head_stride,
                        int64_t ml_plane_stride, const KfaTensor4* out, float* lse, int dtype, void* stream);

/* One backward step for the visiting k / v: scaled fp32 dK, dV stored to (add = 0) or added to
 * (add = 1) dk_acc / dv_acc. stats: as written by kfa_bwd_prepare for the local queries, with
 * stats_head_stride floats between consecutive (b, h) (pass a pointer into the buffer to address a
 * slice of query tiles). */
int kfa_cp_bwd_dkdv_step(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
                         const float* stats, int64_t stats_head_stride, const KfaAcc32* dk_acc,
                         const KfaAcc32* dv_acc, int add, float scale, int block, int dtype, int* dev_status,
                         void* stream);

/* The same for dQ of the local queries. */
int kfa_cp_bwd_dq_step(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
                       const float* stats, int64_t stats_head_stride, const KfaAcc32* dq_acc, int add,
                       float scale, int block, int dtype, int* dev_status, void* stream);

/* grad = acc rounded to 16 bits. */
int kfa_cp_grad_finalize(const KfaAcc32* acc, const KfaTensor4* grad, int dtype, void* stream);

/* Host plumbing for callers whose tensors live in pinned HOST memory (kohakufa_b200/hostio.py): one strided
 * copy of `rows` rows of `row_bytes` bytes between host and device (cudaMemcpy2DAsync on `stream`;
 * to_device != 0: host -> device), e.g. the rows of a group of heads out of [B, S, H, D] storage. No
 * counterpart in the reference, whose callers hold CUDA tensors. */
int kfa_copy_rows(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t row_bytes,
                  int64_t rows, int to_device, void* stream);

/* Diagnostic: the raw scores Q K^T (unscaled, unmasked) as fp32 [B, H, Sq, Skv] (contiguous), produced by
 * the same tensor-core instruction sequence the attention kernels use (one fp32-accumulating MMA per 16
 * elements of the head dim, in ascending order). What comes out is NOT the correctly rounded dot
 * product: the tensor core sums the products of a step with a truncating adder, a few units in the last
 * place away. tests/ use it to compute the accuracy floor of a kernel whose scores come from this
 * hardware. No counterpart in the reference, whose emulation assumes correctly rounded fp32 scores
 * (benchmarks/dinov3_backward.py:236). k may have fewer heads than q (grouped-query attention). */
int kfa_scores(const KfaTensor4* q, const KfaTensor4* k, float* scores, int dtype, int* dev_status,
               void* stream);

/* Hardware self-check of the building blocks (TMA tile load, MMA from shared memory, MMA with a
 * tensor-memory operand, tensor-memory loads / stores) on small fixed matrices. Synchronises.
 * `report` (may be NULL) receives `report_len` bytes of text. No counterpart in the reference. */
int kfa_selftest(char* report, int report_len);

#ifdef __cplusplus
}
#endif

#endif /* KFA_H_ */
