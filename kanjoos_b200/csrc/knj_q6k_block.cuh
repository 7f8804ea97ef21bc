// knj_q6k_block.cuh -- decode-class arithmetic over a block of Q6_K rows staged in shared memory (210-byte
// superblocks: 128 B low nibbles, 64 B high bit pairs, 16 int8 scales, fp16 d; w = d * sc * (q - 32); decoders
// kernels/knj_q4k.h:170-196, CPU dot_q6_k src/loader/dequant.cpp:986-1022). Shared by the stand-alone projection
// kernel (knj_q6k.cu) and the down phase of the whole-stack launch (knj_stack.cu), so both produce the same bits.
#pragma once
#include "knj_common.cuh"
#include "knj_q4k.h"

namespace knj {
namespace q6b {

constexpr int kTok = 8;    // activation rows per pass (accumulators per lane and row)
constexpr int kRows = 64;  // output rows per staged block: a block starts on a 16-byte boundary of the weight stream

// four weights of lane `lane` in half `hf` of a superblock, as sc * (q - 32): positions lane, +32, +64, +96
__device__ __forceinline__ void four(const uint8_t *blk, int hf, int lane, float (&w)[4]) {
  const uint32_t a = blk[64 * hf + lane], b = blk[64 * hf + 32 + lane], h = blk[128 + 32 * hf + lane];
  const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + 8 * hf) + (lane >> 4);
  w[0] = (float)((int)sc[0] * ((int)((a & 15u) | ((h & 3u) << 4)) - 32));
  w[1] = (float)((int)sc[2] * ((int)((b & 15u) | (((h >> 2) & 3u) << 4)) - 32));
  w[2] = (float)((int)sc[4] * ((int)((a >> 4) | (((h >> 4) & 3u) << 4)) - 32));
  w[3] = (float)((int)sc[6] * ((int)((b >> 4) | (((h >> 6) & 3u) << 4)) - 32));
}

// The block's superblocks (rows x row_bytes contiguous bytes at src) into shared memory: 16-byte pieces where the
// start and the length allow it, else 2-byte pieces (rows are 2-byte aligned). All `threads` threads of the CTA.
__device__ __forceinline__ void stage_block(uint8_t *wbuf, const uint8_t *src, int bytes, int tid, int threads) {
  if (((reinterpret_cast<uintptr_t>(src) | (uintptr_t)bytes) & 15u) == 0) {
    for (int i = tid; i < bytes / 16; i += threads) reinterpret_cast<uint4 *>(wbuf)[i] = __ldcs(reinterpret_cast<const uint4 *>(src) + i);
  } else {
    for (int i = tid; i < bytes / 2; i += threads) reinterpret_cast<uint16_t *>(wbuf)[i] = reinterpret_cast<const uint16_t *>(src)[i];
  }
}

// Rows of the staged block against NT staged activation rows (f32 [NT][K] at abuf): a warp takes rows (r, r + WARPS)
// together, so that an activation value read from shared memory meets two weights. store(r, t, value) receives the
// finished sums of row r and activation row t < nt from lane 0. Lane l covers weights l, l+32, l+64, l+96 of every
// 128-weight half; d is applied once per superblock; the warp's partial sums meet in shuffles.
template <int NT, int WARPS, class Store>
__device__ __forceinline__ void rows(const uint8_t *wbuf, const float *abuf, int K, int n_rows, int nt, int lane, int warp, Store store) {
  const int nsb = K / KNJ_QK_K, row_bytes = nsb * KNJ_Q6K_BYTES;
  for (int r = warp; r < n_rows; r += 2 * WARPS) {
    const bool two = r + WARPS < n_rows;
    const int r2 = two ? r + WARPS : r;
    float acc[2][NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[0][t] = acc[1][t] = 0.f;
    for (int sb = 0; sb < nsb; ++sb) {
      const uint8_t *b0 = wbuf + (size_t)r * row_bytes + sb * KNJ_Q6K_BYTES, *b1 = wbuf + (size_t)r2 * row_bytes + sb * KNJ_Q6K_BYTES;
      float part[2][NT];
#pragma unroll
      for (int t = 0; t < NT; ++t) part[0][t] = part[1][t] = 0.f;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        float w0[4], w1[4];
        four(b0, hf, lane, w0);
        four(b1, hf, lane, w1);
        const float *x = abuf + sb * KNJ_QK_K + hf * 128 + lane;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const float *xt = x + (size_t)t * K;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float xv = xt[32 * j];
            part[0][t] = fmaf(w0[j], xv, part[0][t]);
            part[1][t] = fmaf(w1[j], xv, part[1][t]);
          }
        }
      }
      const float d0 = knj_half_bits_to_float((uint16_t)(b0[208] | ((uint16_t)b0[209] << 8)));
      const float d1 = knj_half_bits_to_float((uint16_t)(b1[208] | ((uint16_t)b1[209] << 8)));
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        acc[0][t] = fmaf(d0, part[0][t], acc[0][t]);
        acc[1][t] = fmaf(d1, part[1][t], acc[1][t]);
      }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const float v0 = warp_sum(acc[0][t]), v1 = warp_sum(acc[1][t]);
      if (lane == 0 && t < nt) {
        store(r, t, v0);
        if (two) store(r2, t, v1);
      }
    }
  }
}

// nt activation rows are staged at abuf; rows nt.. up to the next of {1, 2, 4, 8} are zero-filled here (CTA
// barriers inside: every thread of the CTA calls it with the same nt)
template <int WARPS, class Store>
__device__ __forceinline__ void rows_any(const uint8_t *wbuf, float *abuf, int K, int n_rows, int nt, int lane, int warp, Store store) {
  const int tid = warp * 32 + lane;
  if (nt == 1) rows<1, WARPS>(wbuf, abuf, K, n_rows, nt, lane, warp, store);
  else if (nt == 2) rows<2, WARPS>(wbuf, abuf, K, n_rows, nt, lane, warp, store);
  else if (nt <= 4) {
    for (int i = tid; i < (4 - nt) * K; i += WARPS * 32) abuf[(size_t)nt * K + i] = 0.f;
    __syncthreads();
    rows<4, WARPS>(wbuf, abuf, K, n_rows, nt, lane, warp, store);
  } else {
    for (int i = tid; i < (kTok - nt) * K; i += WARPS * 32) abuf[(size_t)nt * K + i] = 0.f;
    __syncthreads();
    rows<kTok, WARPS>(wbuf, abuf, K, n_rows, nt, lane, warp, store);
  }
}

}  // namespace q6b
}  // namespace knj
