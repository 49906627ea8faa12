// C ABI of libkfa.so (declared in include/kfa.h): argument checks, TMA tensor-map encoding and
// kernel launches for the attention forward and backward. No device allocation, no host
// synchronisation (except kfa_selftest), no global mutable state besides per-device "attribute
// already set" flags.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/kfa.h"
#include "kfa_bwd.cuh"
#include "kfa_bwd_fused.cuh"
#include "kfa_fwd.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define KFA_CUDA(expr)                                                                    \
  do {                                                                                    \
    cudaError_t e_ = (expr);                                                              \
    if (e_ != cudaSuccess) return fail(KFA_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static std::atomic<EncodeFn> cached{nullptr};
  EncodeFn f = cached.load();
  if (f) return f;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || !sym)
    return nullptr;
  f = reinterpret_cast<EncodeFn>(sym);
  cached.store(f);
  return f;
}

int check_tensor(const KfaTensor4* t, const char* name) {
  if (!t || !t->ptr) return fail(KFA_ERR_ARG, "%s: null tensor", name);
  if (reinterpret_cast<uintptr_t>(t->ptr) % 16) return fail(KFA_ERR_ARG, "%s: base not 16-byte aligned", name);
  if (t->stride[3] != 1) return fail(KFA_ERR_ARG, "%s: last dimension must be contiguous", name);
  for (int i = 0; i < 3; ++i)
    if (t->shape[i] > 1 && (t->stride[i] % 8 != 0 || t->stride[i] <= 0))
      return fail(KFA_ERR_ARG, "%s: stride[%d]=%lld must be a positive multiple of 8 elements", name, i,
                  static_cast<long long>(t->stride[i]));
  for (int i = 0; i < 4; ++i)
    if (t->shape[i] < 1 || t->shape[i] > 0x7fffffff) return fail(KFA_ERR_ARG, "%s: bad shape[%d]", name, i);
  return KFA_OK;
}

// 4-D tiled map over a [B, H, S, D] view: dims (D, S, H, B), box (C, 128, 1, 1) with C the chunk width of the
// head dim (64, 32 or 16 columns) and the swizzle that spans the box's row (128, 64 or 32 bytes);
// out-of-range rows read as zeros.
int make_map(const KfaTensor4* t, int dtype, CUtensorMap* map, const char* name) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(KFA_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
  const cuuint64_t D = t->shape[3], S = t->shape[2], H = t->shape[1], B = t->shape[0];
  cuuint64_t dims[4] = {D, S, H, B};
  // A dimension of extent 1 never advances: give it any legal stride.
  auto st = [&](int i) -> cuuint64_t {
    const int64_t s = (t->shape[i] > 1) ? t->stride[i] : static_cast<int64_t>(D);
    return static_cast<cuuint64_t>(s) * 2;
  };
  cuuint64_t strides[3] = {st(2), st(1), st(0)};
  const int chunk = kfa::chunk_cols(static_cast<int>(D));
  cuuint32_t box[4] = {static_cast<cuuint32_t>(chunk), 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapSwizzle swizzle =
      chunk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : (chunk == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  CUresult r = enc(map, dtype == KFA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   t->ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(KFA_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", name, (int)r);
  return KFA_OK;
}

int check_qkv(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, int dtype, int block) {
  int rc;
  if ((rc = check_tensor(q, "q")) || (rc = check_tensor(k, "k")) || (rc = check_tensor(v, "v"))) return rc;
  if (dtype != KFA_F16 && dtype != KFA_BF16) return fail(KFA_ERR_ARG, "dtype %d: KFA_F16 or KFA_BF16", dtype);
  const int64_t D = q->shape[3];
  if (D < 16 || D > 128 || D % 16) return fail(KFA_ERR_ARG, "head_dim %lld: a multiple of 16 up to 128", (long long)D);
  for (int i = 0; i < 4; ++i)
    if (k->shape[i] != v->shape[i]) return fail(KFA_ERR_ARG, "k and v shapes differ");
  if (k->shape[0] != q->shape[0] || k->shape[3] != D) return fail(KFA_ERR_ARG, "k / v batch or head_dim differ from q");
  if (q->shape[1] % k->shape[1])
    return fail(KFA_ERR_ARG, "q heads %lld must be a multiple of k / v heads %lld", (long long)q->shape[1],
                (long long)k->shape[1]);
  if (block < 0) return fail(KFA_ERR_ARG, "block %d < 0", block);
  return KFA_OK;
}

int check_like(const KfaTensor4* t, const KfaTensor4* ref, const char* name) {
  int rc = check_tensor(t, name);
  if (rc) return rc;
  for (int i = 0; i < 4; ++i)
    if (t->shape[i] != ref->shape[i]) return fail(KFA_ERR_ARG, "%s: shape differs from its primal", name);
  return KFA_OK;
}

template <typename K>
int set_smem(K kernel, int bytes) {
  KFA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return KFA_OK;
}

constexpr float LOG2E = 1.4426950408889634f;

template <int D, bool BF16, bool MASKW>
int launch_fwd_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const kfa::FwdParams& p,
                 cudaStream_t s) {
  auto kern = kfa::kfa_fwd_kernel<D, BF16, MASKW>;
  constexpr int smem = MASKW ? kfa::FwdCfg<D>::SMEM_BYTES_LIST : kfa::FwdCfg<D>::SMEM_BYTES;
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  const long long grid = static_cast<long long>(p.B) * p.H * p.n_q_tiles;
  if (grid > 0x7fffffffll) return fail(KFA_ERR_ARG, "too many tiles");
  kern<<<static_cast<unsigned>(grid), kfa::FWD_THREADS, smem, s>>>(mq, mk, mv, p);
  KFA_CUDA(cudaGetLastError());
  return KFA_OK;
}

template <int D, bool BF16>
int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const kfa::FwdParams& p,
               cudaStream_t s) {
  return p.mw ? launch_fwd_t<D, BF16, true>(mq, mk, mv, p, s) : launch_fwd_t<D, BF16, false>(mq, mk, mv, p, s);
}

template <int D, bool BF16>
int launch_prepare(const kfa::PrepParams& p, cudaStream_t s) {
  dim3 grid(p.n_q128, p.B * p.H);
  kfa::kfa_bwd_prepare_kernel<D, BF16><<<grid, 128, 0, s>>>(p);
  KFA_CUDA(cudaGetLastError());
  return KFA_OK;
}

template <int D, bool BF16, bool MASKW>
int launch_dkdv_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                  const kfa::BwdParams& p, cudaStream_t s) {
  auto kern = kfa::kfa_bwd_dkdv_kernel<D, BF16, MASKW>;
  constexpr int smem = MASKW ? kfa::BwdCfg<D>::KV_SMEM_BYTES_LIST : kfa::BwdCfg<D>::KV_SMEM_BYTES;
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  const long long grid = static_cast<long long>(p.B) * p.Hkv * p.n_k128;
  if (grid > 0x7fffffffll) return fail(KFA_ERR_ARG, "too many tiles");
  kern<<<static_cast<unsigned>(grid), kfa::BWD_THREADS, smem, s>>>(mq, mk, mv, mdo, p);
  KFA_CUDA(cudaGetLastError());
  return KFA_OK;
}

template <int D, bool BF16>
int launch_dkdv(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                const kfa::BwdParams& p, cudaStream_t s) {
  return p.mwt ? launch_dkdv_t<D, BF16, true>(mq, mk, mv, mdo, p, s) : launch_dkdv_t<D, BF16, false>(mq, mk, mv, mdo, p, s);
}

template <int D, bool BF16, bool MASKW>
int launch_dq_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                const kfa::BwdParams& p, cudaStream_t s) {
  auto kern = kfa::kfa_bwd_dq_kernel<D, BF16, MASKW>;
  constexpr int smem = MASKW ? kfa::BwdCfg<D>::Q_SMEM_BYTES_LIST : kfa::BwdCfg<D>::Q_SMEM_BYTES;
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  const long long grid = static_cast<long long>(p.B) * p.H * p.n_q128;
  if (grid > 0x7fffffffll) return fail(KFA_ERR_ARG, "too many tiles");
  kern<<<static_cast<unsigned>(grid), kfa::BWD_THREADS, smem, s>>>(mq, mk, mv, mdo, p);
  KFA_CUDA(cudaGetLastError());
  return KFA_OK;
}

template <int D, bool BF16>
int launch_dq(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
              const kfa::BwdParams& p, cudaStream_t s) {
  return p.mw ? launch_dq_t<D, BF16, true>(mq, mk, mv, mdo, p, s) : launch_dq_t<D, BF16, false>(mq, mk, mv, mdo, p, s);
}

// Runs `call` with KD = the head dim and KB = (dtype is bf16) as compile-time constants.
#define KFA_DISPATCH_D(KD_, dtype_, call) \
  case KD_: {                             \
    constexpr int KD = KD_;               \
    if ((dtype_) == KFA_F16) {            \
      constexpr bool KB = false;          \
      return call;                        \
    } else {                              \
      constexpr bool KB = true;           \
      return call;                        \
    }                                     \
  }
// The fused backward exists for head dims 64 and 128.
#define KFA_DISPATCH_FUSED(D_, dtype_, call)               \
  do {                                                     \
    switch (D_) {                                          \
      KFA_DISPATCH_D(64, dtype_, call)                     \
      KFA_DISPATCH_D(128, dtype_, call)                    \
      default:                                             \
        return fail(KFA_ERR_ARG, "fused backward: head_dim %d: 64 or 128", (int)(D_)); \
    }                                                      \
  } while (0)
#define KFA_DISPATCH(D_, dtype_, call)                     \
  do {                                                     \
    switch (D_) {                                          \
      KFA_DISPATCH_D(16, dtype_, call)                     \
      KFA_DISPATCH_D(32, dtype_, call)                     \
      KFA_DISPATCH_D(48, dtype_, call)                     \
      KFA_DISPATCH_D(64, dtype_, call)                     \
      KFA_DISPATCH_D(80, dtype_, call)                     \
      KFA_DISPATCH_D(96, dtype_, call)                     \
      KFA_DISPATCH_D(112, dtype_, call)                    \
      KFA_DISPATCH_D(128, dtype_, call)                    \
      default:                                             \
        return fail(KFA_ERR_ARG, "head_dim %d: a multiple of 16 up to 128", (int)(D_)); \
    }                                                      \
  } while (0)

// A packed variable-length batch: n_seqs sequences inside [1, H, T, D] tensors.
struct Varlen {
  const int32_t* cu_q;
  const int32_t* cu_k;
  int n_seqs, max_q, max_k;
};

// What a call may add to the plain problem: a packed variable-length batch, or a boolean mask.
struct Extra {
  const Varlen* vl = nullptr;
  const KfaMaskWords* mw = nullptr;   // words along query rows
  const KfaMaskWords* mwt = nullptr;  // words along key rows
  const KfaMaskTiles* mt = nullptr;   // which 128 x 128 tiles hold a visible pair (optional)
};

int check_tiles(const KfaMaskTiles* t) {
  if (!t) return KFA_OK;
  if (!t->any || t->stride_batch < 0 || t->stride_head < 0) return fail(KFA_ERR_ARG, "mask tiles: null table or negative stride");
  return KFA_OK;
}

// rows: the rows the words must cover; cols: the bits per row (padded to whole 128-wide tiles)
int check_mask(const KfaMaskWords* m, int64_t cols, const char* name) {
  if (!m) return KFA_OK;
  if (!m->words || reinterpret_cast<uintptr_t>(m->words) % 16) return fail(KFA_ERR_ARG, "%s: null or unaligned words", name);
  if (m->stride_row < 4 * ((cols + 127) / 128) || m->stride_row % 4 || m->stride_batch % 4 || m->stride_head % 4 ||
      m->stride_batch < 0 || m->stride_head < 0)
    return fail(KFA_ERR_ARG, "%s: strides must be multiples of 4 words, rows at least %lld words long", name,
                (long long)(4 * ((cols + 127) / 128)));
  return KFA_OK;
}

int check_varlen(const Varlen* vl, const KfaTensor4* q, const KfaTensor4* k) {
  if (!vl) return KFA_OK;
  if (!vl->cu_q || !vl->cu_k) return fail(KFA_ERR_ARG, "cu_seqlens: null pointer");
  if (q->shape[0] != 1 || k->shape[0] != 1) return fail(KFA_ERR_ARG, "packed batches are [1, H, T, D] tensors");
  if (vl->n_seqs < 1 || vl->max_q < 1 || vl->max_k < 1 || vl->max_q > q->shape[2] || vl->max_k > k->shape[2])
    return fail(KFA_ERR_ARG, "packed batch: n_seqs %d, longest sequence %d queries / %d keys, tensors hold %lld / %lld rows",
                vl->n_seqs, vl->max_q, vl->max_k, (long long)q->shape[2], (long long)k->shape[2]);
  return KFA_OK;
}

void fill_bwd_params(kfa::BwdParams& p, const KfaTensor4* q, const KfaTensor4* k, const float* stats, float scale,
                     int block, int* dev_status) {
  std::memset(&p, 0, sizeof(p));
  p.stats = stats;
  p.B = static_cast<int>(q->shape[0]);
  p.H = static_cast<int>(q->shape[1]);
  p.Hkv = static_cast<int>(k->shape[1]);
  p.group = p.H / p.Hkv;
  p.Sq = static_cast<int>(q->shape[2]);
  p.Skv = static_cast<int>(k->shape[2]);
  p.P = block;
  p.c = scale * LOG2E;
  p.scale = scale;
  p.n_q128 = (p.Sq + 127) / 128;
  p.n_k128 = (p.Skv + 127) / 128;
  p.status = dev_status;
  p.stats_sh = static_cast<long long>(p.n_q128) * 384;
}

void apply_extra(kfa::BwdParams& p, const Extra& ex) {
  if (ex.mw) {
    p.mw = ex.mw->words;
    p.mw_sb = ex.mw->stride_batch;
    p.mw_sh = ex.mw->stride_head;
    p.mw_row = static_cast<int>(ex.mw->stride_row);
  }
  if (ex.mwt) {
    p.mwt = ex.mwt->words;
    p.mwt_sb = ex.mwt->stride_batch;
    p.mwt_sh = ex.mwt->stride_head;
    p.mwt_row = static_cast<int>(ex.mwt->stride_row);
  }
  if (ex.mt && ex.mt->any) {
    // the lists of visited tiles live in shared memory: use the table where they fit
    const bool fits_dkdv = static_cast<long long>(p.group) * p.n_q128 <= kfa::BwdCfg<128>::KV_LIST_CAP;
    const bool fits_dq = p.n_k128 <= kfa::BwdCfg<128>::Q_LIST_CAP;
    if (ex.mwt ? fits_dkdv : (ex.mw && fits_dq)) {  // (a call passes the words of ONE of the two kernels)
      p.mt = ex.mt->any;
      p.mt_sb = ex.mt->stride_batch;
      p.mt_sh = ex.mt->stride_head;
      p.mt_row = p.n_k128;
    }
  }
  const Varlen* vl = ex.vl;
  if (!vl) return;
  p.B = vl->n_seqs;
  p.n_q128 = (vl->max_q + 127) / 128;
  p.n_k128 = (vl->max_k + 127) / 128;
  p.stats_sh = static_cast<long long>(p.n_q128) * 384;
  p.cu_q = vl->cu_q;
  p.cu_k = vl->cu_k;
}

int fwd_impl(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out, float* lse,
             const Extra& ex, float scale, int block, int dtype, int* dev_status, void* stream) {
  const Varlen* vl = ex.vl;
  int rc;
  if ((rc = check_qkv(q, k, v, dtype, block)) || (rc = check_like(out, q, "out")) || (rc = check_varlen(vl, q, k)) ||
      (rc = check_mask(ex.mw, k->shape[2], "mask words")))
    return rc;
  if (ex.mw && (block != 0 || vl)) return fail(KFA_ERR_ARG, "a boolean mask excludes block-causal and packed batches");
  if (!lse || !dev_status) return fail(KFA_ERR_ARG, "lse / dev_status: null pointer");
  CUtensorMap mq, mk, mv;
  if ((rc = make_map(q, dtype, &mq, "q")) || (rc = make_map(k, dtype, &mk, "k")) || (rc = make_map(v, dtype, &mv, "v")))
    return rc;
  kfa::FwdParams p;
  std::memset(&p, 0, sizeof(p));
  p.o = out->ptr;
  p.o_sb = out->stride[0];
  p.o_sh = out->stride[1];
  p.o_ss = out->stride[2];
  p.lse = lse;
  p.B = static_cast<int>(q->shape[0]);
  p.H = static_cast<int>(q->shape[1]);
  p.Sq = static_cast<int>(q->shape[2]);
  p.Skv = static_cast<int>(k->shape[2]);
  p.P = block;
  p.c = scale * LOG2E;
  p.n_q_tiles = (p.Sq + 255) / 256;
  p.status = dev_status;
  p.group = static_cast<int>(q->shape[1] / k->shape[1]);
  if (vl) {
    p.B = vl->n_seqs;
    p.n_q_tiles = (vl->max_q + 255) / 256;
    p.cu_q = vl->cu_q;
    p.cu_k = vl->cu_k;
  }
  if (ex.mw) {
    p.mw = ex.mw->words;
    p.mw_sb = ex.mw->stride_batch;
    p.mw_sh = ex.mw->stride_head;
    p.mw_row = static_cast<int>(ex.mw->stride_row);
    const int n_k128 = (p.Skv + 127) / 128;
    if ((rc = check_tiles(ex.mt))) return rc;
    if (ex.mt && n_k128 <= kfa::TILE_LIST_CAP) {  // (longer rows: every key tile is visited)
      p.mt = ex.mt->any;
      p.mt_sb = ex.mt->stride_batch;
      p.mt_sh = ex.mt->stride_head;
      p.mt_row = n_k128;
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(q->shape[3], dtype, (launch_fwd<KD, KB>(mq, mk, mv, p, s)));
}

int prepare_impl(const KfaTensor4* out, const KfaTensor4* dout, const float* lse, float* stats, const Varlen* vl,
                 int dtype, void* stream, float* dq_acc = nullptr) {
  int rc;
  if ((rc = check_tensor(out, "out")) || (rc = check_like(dout, out, "dout"))) return rc;
  if (!lse || !stats) return fail(KFA_ERR_ARG, "lse / stats: null pointer");
  if (dtype != KFA_F16 && dtype != KFA_BF16) return fail(KFA_ERR_ARG, "dtype %d", dtype);
  const int64_t D = out->shape[3];
  if (D < 16 || D > 128 || D % 16) return fail(KFA_ERR_ARG, "head_dim %lld: a multiple of 16 up to 128", (long long)D);
  if (dq_acc && D != 64 && D != 128) return fail(KFA_ERR_ARG, "fused backward: head_dim %lld: 64 or 128", (long long)D);
  kfa::PrepParams p;
  std::memset(&p, 0, sizeof(p));
  p.o = out->ptr;
  p.o_sb = out->stride[0];
  p.o_sh = out->stride[1];
  p.o_ss = out->stride[2];
  p.dout = dout->ptr;
  p.do_sb = dout->stride[0];
  p.do_sh = dout->stride[1];
  p.do_ss = dout->stride[2];
  p.lse = lse;
  p.stats = stats;
  p.dq_acc = dq_acc;
  p.B = static_cast<int>(out->shape[0]);
  p.H = static_cast<int>(out->shape[1]);
  p.Sq = static_cast<int>(out->shape[2]);
  p.n_q128 = (p.Sq + 127) / 128;
  if (vl) {
    p.B = vl->n_seqs;
    p.n_q128 = (vl->max_q + 127) / 128;
    p.cu_q = vl->cu_q;
  }
  if (static_cast<long long>(p.B) * p.H > 65535) return fail(KFA_ERR_ARG, "B * H > 65535");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(D, dtype, (launch_prepare<KD, KB>(p, s)));
}

int dkdv_impl(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
              const float* stats, const KfaTensor4* dk, const KfaTensor4* dv, const Extra& ex, float scale, int block,
              int dtype, int* dev_status, void* stream) {
  int rc;
  if ((rc = check_qkv(q, k, v, dtype, block)) || (rc = check_like(dout, q, "dout")) ||
      (rc = check_like(dk, k, "dk")) || (rc = check_like(dv, v, "dv")) || (rc = check_varlen(ex.vl, q, k)) ||
      (rc = check_mask(ex.mwt, q->shape[2], "transposed mask words")))
    return rc;
  if (ex.mwt && (block != 0 || ex.vl)) return fail(KFA_ERR_ARG, "a boolean mask excludes block-causal and packed batches");
  if (!stats || !dev_status) return fail(KFA_ERR_ARG, "stats / dev_status: null pointer");
  CUtensorMap mq, mk, mv, mdo;
  if ((rc = make_map(q, dtype, &mq, "q")) || (rc = make_map(k, dtype, &mk, "k")) ||
      (rc = make_map(v, dtype, &mv, "v")) || (rc = make_map(dout, dtype, &mdo, "dout")))
    return rc;
  kfa::BwdParams p;
  fill_bwd_params(p, q, k, stats, scale, block, dev_status);
  apply_extra(p, ex);
  p.dk = dk->ptr;
  p.dk_sb = dk->stride[0];
  p.dk_sh = dk->stride[1];
  p.dk_ss = dk->stride[2];
  p.dv = dv->ptr;
  p.dv_sb = dv->stride[0];
  p.dv_sh = dv->stride[1];
  p.dv_ss = dv->stride[2];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(q->shape[3], dtype, (launch_dkdv<KD, KB>(mq, mk, mv, mdo, p, s)));
}

int dq_impl(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout, const float* stats,
            const KfaTensor4* dq, const Extra& ex, float scale, int block, int dtype, int* dev_status, void* stream) {
  int rc;
  if ((rc = check_qkv(q, k, v, dtype, block)) || (rc = check_like(dout, q, "dout")) ||
      (rc = check_like(dq, q, "dq")) || (rc = check_varlen(ex.vl, q, k)) ||
      (rc = check_mask(ex.mw, k->shape[2], "mask words")))
    return rc;
  if (ex.mw && (block != 0 || ex.vl)) return fail(KFA_ERR_ARG, "a boolean mask excludes block-causal and packed batches");
  if (!stats || !dev_status) return fail(KFA_ERR_ARG, "stats / dev_status: null pointer");
  CUtensorMap mq, mk, mv, mdo;
  if ((rc = make_map(q, dtype, &mq, "q")) || (rc = make_map(k, dtype, &mk, "k")) ||
      (rc = make_map(v, dtype, &mv, "v")) || (rc = make_map(dout, dtype, &mdo, "dout")))
    return rc;
  kfa::BwdParams p;
  fill_bwd_params(p, q, k, stats, scale, block, dev_status);
  apply_extra(p, ex);
  p.dq = dq->ptr;
  p.dq_sb = dq->stride[0];
  p.dq_sh = dq->stride[1];
  p.dq_ss = dq->stride[2];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(q->shape[3], dtype, (launch_dq<KD, KB>(mq, mk, mv, mdo, p, s)));
}


template <int D, bool BF16>
int launch_fused(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                 const kfa::BwdParams& p, float* dq_acc, cudaStream_t s) {
  auto kern = kfa::kfa_bwd_fused_kernel<D, BF16>;
  constexpr int smem = kfa::FusedCfg<D>::SMEM_BYTES;
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  const long long grid = static_cast<long long>(p.B) * p.Hkv * p.n_k128;
  if (grid > 0x7fffffffll) return fail(KFA_ERR_ARG, "too many tiles");
  kern<<<static_cast<unsigned>(grid), kfa::FUSED_THREADS, smem, s>>>(mq, mk, mv, mdo, p, dq_acc);
  KFA_CUDA(cudaGetLastError());
  return KFA_OK;
}

template <int D, bool BF16>
int launch_dq_convert(const float* dq_acc, const KfaTensor4* dq, float scale, const int* status, cudaStream_t s) {
  const int H = static_cast<int>(dq->shape[1]), Sq = static_cast<int>(dq->shape[2]);
  auto conv = kfa::kfa_bwd_dq_convert_kernel<D, BF16>;
  conv<<<dim3((Sq + 127) / 128, static_cast<unsigned>(dq->shape[0] * H)), 256, 0, s>>>(
      dq_acc, dq->ptr, dq->stride[0], dq->stride[1], dq->stride[2], H, Sq, scale, status);
  KFA_CUDA(cudaGetLastError());
  return KFA_OK;
}

int convert_impl(const float* dq_acc, const KfaTensor4* dq, float scale, int dtype, const int* dev_status, void* stream) {
  int rc;
  if ((rc = check_tensor(dq, "dq"))) return rc;
  if (!dq_acc || !dev_status) return fail(KFA_ERR_ARG, "dq_acc / dev_status: null pointer");
  if (dtype != KFA_F16 && dtype != KFA_BF16) return fail(KFA_ERR_ARG, "dtype %d", dtype);
  const int64_t D = dq->shape[3];
  if (D != 64 && D != 128) return fail(KFA_ERR_ARG, "head_dim %lld: 64 or 128", (long long)D);
  if (dq->shape[0] * dq->shape[1] > 65535) return fail(KFA_ERR_ARG, "B * H > 65535");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH_FUSED(D, dtype, (launch_dq_convert<KD, KB>(dq_acc, dq, scale, dev_status, s)));
}

int fused_impl(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
               const float* stats, float* dq_acc, const KfaTensor4* dk, const KfaTensor4* dv, float scale, int block,
               int dtype, int* dev_status, void* stream) {
  int rc;
  if ((rc = check_qkv(q, k, v, dtype, block)) || (rc = check_like(dout, q, "dout")) || (rc = check_like(dk, k, "dk")) ||
      (rc = check_like(dv, v, "dv")))
    return rc;
  if (!stats || !dq_acc || !dev_status) return fail(KFA_ERR_ARG, "stats / dq_acc / dev_status: null pointer");
  if (reinterpret_cast<uintptr_t>(dq_acc) % 16) return fail(KFA_ERR_ARG, "dq_acc: not 16-byte aligned");
  CUtensorMap mq, mk, mv, mdo;
  if ((rc = make_map(q, dtype, &mq, "q")) || (rc = make_map(k, dtype, &mk, "k")) ||
      (rc = make_map(v, dtype, &mv, "v")) || (rc = make_map(dout, dtype, &mdo, "dout")))
    return rc;
  kfa::BwdParams p;
  fill_bwd_params(p, q, k, stats, scale, block, dev_status);
  p.dk = dk->ptr;
  p.dk_sb = dk->stride[0];
  p.dk_sh = dk->stride[1];
  p.dk_ss = dk->stride[2];
  p.dv = dv->ptr;
  p.dv_sb = dv->stride[0];
  p.dv_sh = dv->stride[1];
  p.dv_ss = dv->stride[2];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH_FUSED(q->shape[3], dtype, (launch_fused<KD, KB>(mq, mk, mv, mdo, p, dq_acc, s)));
}

}  // namespace

extern "C" {

int kfa_abi_version(void) { return KFA_ABI_VERSION; }

const char* kfa_last_error(void) { return g_err; }

int64_t kfa_bwd_stats_bytes(int64_t B, int64_t H, int64_t Sq) {
  return B * H * ((Sq + 127) / 128) * 3 * 128 * 4;
}

int kfa_fwd(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out, float* lse,
            float scale, int block, int dtype, int* dev_status, void* stream) {
  return fwd_impl(q, k, v, out, lse, Extra{}, scale, block, dtype, dev_status, stream);
}

int kfa_bwd_prepare(const KfaTensor4* out, const KfaTensor4* dout, const float* lse, float* stats, int dtype,
                    void* stream) {
  return prepare_impl(out, dout, lse, stats, nullptr, dtype, stream);
}

int kfa_bwd_dkdv(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
                 const float* stats, const KfaTensor4* dk, const KfaTensor4* dv, float scale, int block, int dtype,
                 int* dev_status, void* stream) {
  return dkdv_impl(q, k, v, dout, stats, dk, dv, Extra{}, scale, block, dtype, dev_status, stream);
}

int kfa_bwd_dq(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
               const float* stats, const KfaTensor4* dq, float scale, int block, int dtype, int* dev_status,
               void* stream) {
  return dq_impl(q, k, v, dout, stats, dq, Extra{}, scale, block, dtype, dev_status, stream);
}

int kfa_fwd_varlen(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out, float* lse,
                   const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int n_seqs, int max_q, int max_k,
                   float scale, int block, int dtype, int* dev_status, void* stream) {
  const Varlen vl{cu_seqlens_q, cu_seqlens_k, n_seqs, max_q, max_k};
  Extra ex;
  ex.vl = &vl;
  return fwd_impl(q, k, v, out, lse, ex, scale, block, dtype, dev_status, stream);
}

int kfa_fwd_masked(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out, float* lse,
                   const KfaMaskWords* words, const KfaMaskTiles* tiles, float scale, int dtype, int* dev_status,
                   void* stream) {
  if (!words) return fail(KFA_ERR_ARG, "kfa_fwd_masked: null mask");
  Extra ex;
  ex.mw = words;
  ex.mt = tiles;
  return fwd_impl(q, k, v, out, lse, ex, scale, 0, dtype, dev_status, stream);
}

int kfa_bwd_masked(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
                   const KfaTensor4* dout, const float* lse, float* stats, const KfaTensor4* dq, const KfaTensor4* dk,
                   const KfaTensor4* dv, const KfaMaskWords* words, const KfaMaskWords* words_t,
                   const KfaMaskTiles* tiles, float scale, int dtype, int* dev_status, void* stream) {
  if (!words || !words_t) return fail(KFA_ERR_ARG, "kfa_bwd_masked: null mask");
  Extra ex_kv, ex_q;
  ex_kv.mwt = words_t;
  ex_q.mw = words;
  ex_kv.mt = ex_q.mt = tiles;
  int rc;
  if ((rc = check_like(out, q, "out")) || (rc = check_tiles(tiles))) return rc;
  if ((rc = prepare_impl(out, dout, lse, stats, nullptr, dtype, stream))) return rc;
  if ((rc = dkdv_impl(q, k, v, dout, stats, dk, dv, ex_kv, scale, 0, dtype, dev_status, stream))) return rc;
  return dq_impl(q, k, v, dout, stats, dq, ex_q, scale, 0, dtype, dev_status, stream);
}

int kfa_bwd_varlen(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
                   const KfaTensor4* dout, const float* lse, float* stats, const KfaTensor4* dq, const KfaTensor4* dk,
                   const KfaTensor4* dv, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int n_seqs,
                   int max_q, int max_k, float scale, int block, int dtype, int* dev_status, void* stream) {
  const Varlen vl{cu_seqlens_q, cu_seqlens_k, n_seqs, max_q, max_k};
  int rc;
  if ((rc = check_like(out, q, "out"))) return rc;
  if ((rc = prepare_impl(out, dout, lse, stats, &vl, dtype, stream))) return rc;
  Extra ex;
  ex.vl = &vl;
  if ((rc = dkdv_impl(q, k, v, dout, stats, dk, dv, ex, scale, block, dtype, dev_status, stream))) return rc;
  return dq_impl(q, k, v, dout, stats, dq, ex, scale, block, dtype, dev_status, stream);
}

int kfa_bwd(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
            const KfaTensor4* dout, const float* lse, float* stats, const KfaTensor4* dq, const KfaTensor4* dk,
            const KfaTensor4* dv, float scale, int block, int dtype, int* dev_status, void* stream) {
  int rc;
  if ((rc = check_like(out, q, "out"))) return rc;
  if ((rc = kfa_bwd_prepare(out, dout, lse, stats, dtype, stream))) return rc;
  if ((rc = kfa_bwd_dkdv(q, k, v, dout, stats, dk, dv, scale, block, dtype, dev_status, stream))) return rc;
  return kfa_bwd_dq(q, k, v, dout, stats, dq, scale, block, dtype, dev_status, stream);
}

#ifdef KFA_TRACE
int kfa_trace_read(long long* out) {
  return cudaMemcpyFromSymbol(out, kfa::kfa_trace, sizeof(kfa::kfa_trace)) == cudaSuccess ? 0 : 1;
}
#endif

int kfa_copy_rows(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t row_bytes, int64_t rows,
                  int to_device, void* stream) {
  if (!dst || !src || row_bytes <= 0 || rows <= 0 || dst_pitch < row_bytes || src_pitch < row_bytes)
    return fail(KFA_ERR_ARG, "kfa_copy_rows: null pointer or pitch shorter than a row");
  KFA_CUDA(cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch), src, static_cast<size_t>(src_pitch),
                             static_cast<size_t>(row_bytes), static_cast<size_t>(rows),
                             to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                             static_cast<cudaStream_t>(stream)));
  return KFA_OK;
}

int64_t kfa_bwd_dq_acc_bytes(int64_t B, int64_t H, int64_t Sq, int64_t D) {
  return B * H * ((Sq + 127) / 128) * 128 * D * 4;
}

int kfa_bwd_prepare_fused(const KfaTensor4* out, const KfaTensor4* dout, const float* lse, float* stats, float* dq_acc,
                          int dtype, void* stream) {
  if (!dq_acc) return fail(KFA_ERR_ARG, "dq_acc: null pointer");
  return prepare_impl(out, dout, lse, stats, nullptr, dtype, stream, dq_acc);
}

int kfa_bwd_fused_main(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
                       const float* stats, float* dq_acc, const KfaTensor4* dk, const KfaTensor4* dv, float scale,
                       int block, int dtype, int* dev_status, void* stream) {
  return fused_impl(q, k, v, dout, stats, dq_acc, dk, dv, scale, block, dtype, dev_status, stream);
}

int kfa_bwd_dq_convert(const float* dq_acc, const KfaTensor4* dq, float scale, int dtype, const int* dev_status,
                       void* stream) {
  return convert_impl(dq_acc, dq, scale, dtype, dev_status, stream);
}

int kfa_bwd_fused(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* out,
                  const KfaTensor4* dout, const float* lse, float* stats, float* dq_acc, const KfaTensor4* dq,
                  const KfaTensor4* dk, const KfaTensor4* dv, float scale, int block, int dtype, int* dev_status,
                  void* stream) {
  int rc;
  if ((rc = check_like(out, q, "out")) || (rc = check_like(dq, q, "dq"))) return rc;
  if (static_cast<long long>(q->shape[0]) * q->shape[1] > 65535) return fail(KFA_ERR_ARG, "B * H > 65535");
  if ((rc = kfa_bwd_prepare_fused(out, dout, lse, stats, dq_acc, dtype, stream))) return rc;
  if ((rc = fused_impl(q, k, v, dout, stats, dq_acc, dk, dv, scale, block, dtype, dev_status, stream))) return rc;
  return convert_impl(dq_acc, dq, scale, dtype, dev_status, stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// kfa_bwd_static_scratch: the backward for callers that cannot hand over scratch memory.
// The per-row statistics (the only scratch of the backward) live in this fixed array instead of a
// caller buffer. It exists once per GPU that loads the library, for the life of the process.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr long long kStaticStatsFloats = KFA_STATIC_SCRATCH_BYTES / 4;
static __device__ __align__(256) float g_static_stats[kStaticStatsFloats];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
float* g_static_stats_addr[kMaxDevices] = {};  // device address of g_static_stats, per device

// The array's name is only a host-side handle: the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_stats_address(float** out) {
  int dev = -1;
  KFA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(KFA_ERR_ARG, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_stats_addr[dev]) {
    void* addr = nullptr;
    KFA_CUDA(cudaGetSymbolAddress(&addr, g_static_stats));
    if (!addr) return fail(KFA_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_static_stats_addr[dev] = static_cast<float*>(addr);
  }
  *out = g_static_stats_addr[dev];
  return KFA_OK;
}

}  // namespace

extern "C" int kfa_bwd_static_scratch(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v,
                                      const KfaTensor4* out, const KfaTensor4* dout, const float* lse,
                                      const KfaTensor4* dq, const KfaTensor4* dk, const KfaTensor4* dv,
                                      float scale, int block, int dtype, int* dev_status, void* stream) {
  int rc = check_tensor(q, "q");
  if (rc) return rc;
  const long long need = kfa_bwd_stats_bytes(q->shape[0], q->shape[1], q->shape[2]);
  if (need > KFA_STATIC_SCRATCH_BYTES)
    return fail(KFA_ERR_ARG,
                "kfa_bwd_static_scratch: B*H*ceil(Sq/128) = %lld tiles need %lld bytes of statistics, the built-in "
                "scratch holds %lld (%lld tiles): use kfa_bwd with a caller buffer",
                need / 1536, need, (long long)KFA_STATIC_SCRATCH_BYTES, (long long)KFA_STATIC_SCRATCH_BYTES / 1536);
  float* stats = nullptr;
  if ((rc = static_stats_address(&stats))) return rc;
  // Every float of every tile used is rewritten by the prepare step: nothing has to start at zero.
  return kfa_bwd(q, k, v, out, dout, lse, stats, dq, dk, dv, scale, block, dtype, dev_status, stream);
}

#include "kfa_cp.cuh"
#include "kfa_mask.cuh"
#include "kfa_scores.cuh"
#include "kfa_selftest.cuh"

