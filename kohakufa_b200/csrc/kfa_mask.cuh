// Boolean attention masks, packed for the kernels: 32 keys per 32-bit word along each query row
// (`words`, read by the forward and the dQ kernel, whose threads own query rows) and 32 queries per word
// along each key row (`words_t`, read by the dK / dV kernel, whose threads own key rows). Bit c % 32 of
// word c / 32 is key (query) c; rows are padded with zero bits to whole 128-wide tiles, so a tile's four
// words never run past a row and padded keys / queries are hidden without a length check.
// Same word format as the reference's packing (src/kohakufa/mask.py:32-72). Instead of the reference's
// per-tile any / all classes and host-built tile lists (mask.py:74-122) the packing marks, in one int per
// (128 queries x 128 keys) tile, whether the tile holds any visible pair; every CTA builds the list of
// tiles it visits from that table in shared memory, and a warp whose bits are all set skips the masking
// code.
// Included at the end of kfa_api.cu (uses its helpers).
#pragma once

namespace kfa {

// One warp packs a 32 x 32 tile of the mask: ballots over keys give the rows' words, ballots over
// queries (through shared memory) the transposed ones. Grid: (ceil(cols32), ceil(rows32), slices).
__global__ void __launch_bounds__(128) kfa_pack_mask_kernel(const uint8_t* mask, long long m_sb, long long m_sh,
                                                            long long m_sr, long long m_sc, int Hm, int Sq, int Skv,
                                                            int* words, int wq /*ints per row of words*/, int* words_t,
                                                            int wk /*ints per row of words_t*/, int* tiles) {
  __shared__ uint8_t tile[4][32][33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cb = blockIdx.x * 4 + warp;  // 32-key block
  const int rb = blockIdx.y;             // 32-query block
  const int slice = blockIdx.z;
  const int b = slice / Hm, h = slice % Hm;
  const bool live = cb < wq;  // (wq = 4 * ceil(Skv / 128) >= ceil(Skv / 32))
  const uint8_t* src = mask + b * m_sb + h * m_sh;
  const int col = cb * 32 + lane;
  if (live) {
    for (int r = 0; r < 32; ++r) {
      const int row = rb * 32 + r;
      uint8_t bit = 0;
      if (row < Sq && col < Skv) bit = src[row * m_sr + col * m_sc] != 0;
      tile[warp][r][lane] = bit;
      const unsigned w = __ballot_sync(0xffffffffu, bit != 0);
      if (lane == 0 && row < Sq) words[(static_cast<long long>(slice) * Sq + row) * wq + cb] = static_cast<int>(w);
    }
  }
  __syncwarp();
  if (live && tiles != nullptr) {  // any bit set in this 32 x 32 block: mark its 128 x 128 tile
    bool some = false;
    for (int r = 0; r < 32; ++r) some |= tile[warp][r][lane] != 0;
    if (__any_sync(0xffffffffu, some) && lane == 0)
      atomicOr(tiles + (static_cast<long long>(slice) * (wk / 4) + rb / 4) * (wq / 4) + cb / 4, 1);
  }
  if (live) {
    for (int c = 0; c < 32; ++c) {
      const int key = cb * 32 + c;
      const unsigned w = __ballot_sync(0xffffffffu, tile[warp][lane][c] != 0);  // lane = query within the block
      if (lane == 0 && key < Skv && rb < wk) words_t[(static_cast<long long>(slice) * Skv + key) * wk + rb] = static_cast<int>(w);
    }
  }
}

// Zero fill of the word columns the pack kernel's grid does not reach (rows of words_t are padded to
// whole 128-query tiles: 4 * ceil(Sq / 128) ints, of which ceil(Sq / 32) are written above).
__global__ void kfa_zero_words_kernel(int* words, long long rows, int width, int first) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const int pad = width - first;
  if (pad <= 0 || i >= rows * pad) return;
  words[(i / pad) * width + first + i % pad] = 0;
}

}  // namespace kfa

extern "C" int kfa_pack_mask(const void* mask, const int64_t* mask_stride, int mask_batch, int mask_heads, int Sq,
                             int Skv, int32_t* words, int32_t* words_t, int32_t* tiles, void* stream) {
  if (!mask || !mask_stride || !words || !words_t) return fail(KFA_ERR_ARG, "kfa_pack_mask: null pointer");
  if (mask_batch < 1 || mask_heads < 1 || Sq < 1 || Skv < 1) return fail(KFA_ERR_ARG, "kfa_pack_mask: empty mask");
  const int wq = 4 * ((Skv + 127) / 128), wk = 4 * ((Sq + 127) / 128);
  const int slices = mask_batch * mask_heads;
  if (slices > 65535 || (Sq + 31) / 32 > 65535) return fail(KFA_ERR_ARG, "kfa_pack_mask: mask too large for one launch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((wq + 3) / 4, (Sq + 31) / 32, slices);
  kfa::kfa_pack_mask_kernel<<<grid, 128, 0, s>>>(static_cast<const uint8_t*>(mask), mask_stride[0], mask_stride[1],
                                                 mask_stride[2], mask_stride[3], mask_heads, Sq, Skv, words, wq,
                                                 words_t, wk, tiles);
  KFA_CUDA(cudaGetLastError());
  const int written = (Sq + 31) / 32;
  if (wk > written) {
    const long long n = static_cast<long long>(slices) * Skv * (wk - written);
    kfa::kfa_zero_words_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(
        words_t, static_cast<long long>(slices) * Skv, wk, written);
    KFA_CUDA(cudaGetLastError());
  }
  return KFA_OK;
}
