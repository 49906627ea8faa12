// Context-parallel building blocks: one attention problem whose sequence is spread over several
// GPUs is computed as a sequence of (local queries) x (visiting keys / values) steps. These entry
// points run one such step with the ordinary kernels and keep everything that crosses steps in fp32:
//   forward   the unnormalised O accumulator with its (m, l) per row (never a fused lse); a step
//             merges its partial result into the carry by shifting both to the common row max;
//             kfa_cp_fwd_finalize normalises and rounds once at the end;
//   backward  fp32 dQ accumulates at home, fp32 dK / dV partials travel with their K / V; they are
//             rounded once by kfa_cp_grad_finalize.
// The reference is single-GPU: these functions have no counterpart there. Included at the end of
// kfa_api.cu (uses its helpers).
#pragma once

namespace kfa {

// out16[row] = acc32[row] * (1 / l[row]) (l == nullptr: no scaling); optionally lse planes (m, log2 l).
template <int D, bool BF16>
__global__ void __launch_bounds__(256) kfa_cp_finalize_kernel(const float* acc, long long acc_sh, const float* ml,
                                                              long long ml_sh, long long ml_plane, void* out,
                                                              long long o_sb, long long o_sh, long long o_ss,
                                                              float* lse, int H, int S) {
  constexpr int LPR = D / 8;  // lanes per row, 8 elements each
  const int bh = blockIdx.y;
  const int b = bh / H, h = bh % H;
  const int row = blockIdx.x * (256 / LPR) + threadIdx.x / LPR;
  const int vec = threadIdx.x % LPR;
  if (row >= S) return;
  float inv = 1.0f;
  if (ml != nullptr) {
    const float m = ml[bh * ml_sh + row], l = ml[bh * ml_sh + ml_plane + row];
    inv = 1.0f / l;
    if (lse != nullptr && vec == 0) {
      lse[static_cast<long long>(bh) * 2 * S + row] = m;
      lse[static_cast<long long>(bh) * 2 * S + S + row] = log2f(l);
    }
  }
  const float* src = acc + bh * acc_sh + static_cast<long long>(row) * D + vec * 8;
  const float4 a0 = *reinterpret_cast<const float4*>(src);
  const float4 a1 = *reinterpret_cast<const float4*>(src + 4);
  uint4 w;
  w.x = pack16<BF16>(a0.x * inv, a0.y * inv);
  w.y = pack16<BF16>(a0.z * inv, a0.w * inv);
  w.z = pack16<BF16>(a1.x * inv, a1.y * inv);
  w.w = pack16<BF16>(a1.z * inv, a1.w * inv);
  uint8_t* dst = reinterpret_cast<uint8_t*>(out) + 2 * (b * o_sb + h * o_sh + static_cast<long long>(row) * o_ss + vec * 8);
  *reinterpret_cast<uint4*>(dst) = w;
}

}  // namespace kfa

namespace {

int check_acc(const KfaAcc32* a, const char* name) {
  if (!a || !a->ptr) return fail(KFA_ERR_ARG, "%s: null accumulator", name);
  if (reinterpret_cast<uintptr_t>(a->ptr) % 16 || a->head_stride % 4)
    return fail(KFA_ERR_ARG, "%s: accumulator must be 16-byte aligned with a head stride that is a multiple of 4", name);
  return KFA_OK;
}

template <int D, bool BF16>
int launch_finalize(const KfaAcc32* acc, const float* ml, long long ml_sh, long long ml_plane, const KfaTensor4* out,
                    float* lse, cudaStream_t s) {
  const int S = static_cast<int>(out->shape[2]);
  const int BH = static_cast<int>(out->shape[0] * out->shape[1]);
  constexpr int rows_per_block = 256 / (D / 8);
  dim3 grid((S + rows_per_block - 1) / rows_per_block, BH);
  kfa::kfa_cp_finalize_kernel<D, BF16><<<grid, 256, 0, s>>>(acc->ptr, acc->head_stride, ml, ml_sh, ml_plane, out->ptr,
                                                            out->stride[0], out->stride[1], out->stride[2], lse,
                                                            static_cast<int>(out->shape[1]), S);
  KFA_CUDA(cudaGetLastError());
  return KFA_OK;
}

}  // namespace

extern "C" {

int kfa_cp_fwd_step(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaAcc32* o_acc, float* ml,
                    int64_t ml_head_stride, int64_t ml_plane_stride, int merge, float scale, int block, int dtype,
                    int* dev_status, void* stream) {
  int rc;
  if ((rc = check_qkv(q, k, v, dtype, block)) || (rc = check_acc(o_acc, "o_acc"))) return rc;
  if (!ml || !dev_status) return fail(KFA_ERR_ARG, "ml / dev_status: null pointer");
  CUtensorMap mq, mk, mv;
  if ((rc = make_map(q, dtype, &mq, "q")) || (rc = make_map(k, dtype, &mk, "k")) || (rc = make_map(v, dtype, &mv, "v")))
    return rc;
  kfa::FwdParams p;
  std::memset(&p, 0, sizeof(p));
  p.B = static_cast<int>(q->shape[0]);
  p.H = static_cast<int>(q->shape[1]);
  p.Sq = static_cast<int>(q->shape[2]);
  p.Skv = static_cast<int>(k->shape[2]);
  p.P = block;
  p.c = scale * LOG2E;
  p.n_q_tiles = (p.Sq + 255) / 256;
  p.status = dev_status;
  p.group = static_cast<int>(q->shape[1] / k->shape[1]);
  p.mode = merge ? 2 : 1;
  p.o_acc = o_acc->ptr;
  p.oa_sh = o_acc->head_stride;
  p.ml = ml;
  p.ml_sh = ml_head_stride;
  p.ml_plane = ml_plane_stride;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(q->shape[3], dtype, (launch_fwd<KD, KB>(mq, mk, mv, p, s)));
}

int kfa_cp_fwd_finalize(const KfaAcc32* o_acc, const float* ml, int64_t ml_head_stride, int64_t ml_plane_stride,
                        const KfaTensor4* out, float* lse, int dtype, void* stream) {
  int rc;
  if ((rc = check_acc(o_acc, "o_acc")) || (rc = check_tensor(out, "out"))) return rc;
  if (!ml || !lse) return fail(KFA_ERR_ARG, "ml / lse: null pointer");
  const int64_t D = out->shape[3];
  if (D != 64 && D != 128) return fail(KFA_ERR_ARG, "head_dim %lld: 64 or 128", (long long)D);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(D, dtype, (launch_finalize<KD, KB>(o_acc, ml, ml_head_stride, ml_plane_stride, out, lse, s)));
}

int kfa_cp_grad_finalize(const KfaAcc32* acc, const KfaTensor4* grad, int dtype, void* stream) {
  int rc;
  if ((rc = check_acc(acc, "acc")) || (rc = check_tensor(grad, "grad"))) return rc;
  const int64_t D = grad->shape[3];
  if (D != 64 && D != 128) return fail(KFA_ERR_ARG, "head_dim %lld: 64 or 128", (long long)D);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(D, dtype, (launch_finalize<KD, KB>(acc, nullptr, 0, 0, grad, nullptr, s)));
}

int kfa_cp_bwd_dkdv_step(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
                         const float* stats, int64_t stats_head_stride, const KfaAcc32* dk_acc, const KfaAcc32* dv_acc,
                         int add, float scale, int block, int dtype, int* dev_status, void* stream) {
  int rc;
  if ((rc = check_qkv(q, k, v, dtype, block)) || (rc = check_like(dout, q, "dout")) ||
      (rc = check_acc(dk_acc, "dk_acc")) || (rc = check_acc(dv_acc, "dv_acc")))
    return rc;
  if (!stats || !dev_status) return fail(KFA_ERR_ARG, "stats / dev_status: null pointer");
  CUtensorMap mq, mk, mv, mdo;
  if ((rc = make_map(q, dtype, &mq, "q")) || (rc = make_map(k, dtype, &mk, "k")) ||
      (rc = make_map(v, dtype, &mv, "v")) || (rc = make_map(dout, dtype, &mdo, "dout")))
    return rc;
  kfa::BwdParams p;
  fill_bwd_params(p, q, k, stats, scale, block, dev_status);
  p.stats_sh = stats_head_stride;
  p.acc_mode = add ? 2 : 1;
  p.dk32 = dk_acc->ptr;
  p.dk32_sh = dk_acc->head_stride;
  p.dv32 = dv_acc->ptr;
  p.dv32_sh = dv_acc->head_stride;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(q->shape[3], dtype, (launch_dkdv<KD, KB>(mq, mk, mv, mdo, p, s)));
}

int kfa_cp_bwd_dq_step(const KfaTensor4* q, const KfaTensor4* k, const KfaTensor4* v, const KfaTensor4* dout,
                       const float* stats, int64_t stats_head_stride, const KfaAcc32* dq_acc, int add, float scale,
                       int block, int dtype, int* dev_status, void* stream) {
  int rc;
  if ((rc = check_qkv(q, k, v, dtype, block)) || (rc = check_like(dout, q, "dout")) || (rc = check_acc(dq_acc, "dq_acc")))
    return rc;
  if (!stats || !dev_status) return fail(KFA_ERR_ARG, "stats / dev_status: null pointer");
  CUtensorMap mq, mk, mv, mdo;
  if ((rc = make_map(q, dtype, &mq, "q")) || (rc = make_map(k, dtype, &mk, "k")) ||
      (rc = make_map(v, dtype, &mv, "v")) || (rc = make_map(dout, dtype, &mdo, "dout")))
    return rc;
  kfa::BwdParams p;
  fill_bwd_params(p, q, k, stats, scale, block, dev_status);
  p.stats_sh = stats_head_stride;
  p.acc_mode = add ? 2 : 1;
  p.dq32 = dq_acc->ptr;
  p.dq32_sh = dq_acc->head_stride;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KFA_DISPATCH(q->shape[3], dtype, (launch_dq<KD, KB>(mq, mk, mv, mdo, p, s)));
}

}  // extern "C"
