// knj_q6k_block.cuh -- decode-class arithmetic over a block of Q6_K rows staged in shared memory (210-byte
// superblocks: 128 B low nibbles, 64 B high bit pairs, 16 int8 scales, fp16 d; w = d * sc * (q - 32); decoders
// kernels/knj_q4k.h:170-196, CPU dot_q6_k src/loader/dequant.cpp:986-1022). Shared by the stand-alone projection
// kernel (knj_q6k.cu) and the down phase of the whole-stack launch (knj_stack.cu), so both produce the same bits.
#pragma once
#include "knj_common.cuh"
#include "knj_q4k.h"

namespace knj {
namespace q6b {

constexpr int kTok = 8;    // activation rows per pass: two MMA column groups of four
constexpr int kRows = 64;  // output rows per staged block: a block starts on a 16-byte boundary of the weight stream

// The block's superblocks (rows x row_bytes contiguous bytes at src) into shared memory: 16-byte pieces where the
// start and the length allow it, else 2-byte pieces (rows are 2-byte aligned). All `threads` threads of the CTA.
__device__ __forceinline__ void stage_block(uint8_t *wbuf, const uint8_t *src, int bytes, int tid, int threads) {
  if (((reinterpret_cast<uintptr_t>(src) | (uintptr_t)bytes) & 15u) == 0) {
    for (int i = tid; i < bytes / 16; i += threads) reinterpret_cast<uint4 *>(wbuf)[i] = __ldcs(reinterpret_cast<const uint4 *>(src) + i);
  } else {
    for (int i = tid; i < bytes / 2; i += threads) reinterpret_cast<uint16_t *>(wbuf)[i] = reinterpret_cast<const uint16_t *>(src)[i];
  }
}

// The same by one bulk copy that completes on `bar` (one thread calls it; the others wait on the barrier): for blocks
// that start on a 16-byte boundary and are a multiple of 16 bytes long (bulk_ok). Earlier reads of the buffer by
// this CTA must have been ordered before the call by a CTA barrier.
__device__ __forceinline__ bool bulk_ok(const uint8_t *src, int bytes) {
  return ((reinterpret_cast<uintptr_t>(src) | (uintptr_t)bytes) & 15u) == 0;
}
__device__ __forceinline__ void stage_block_bulk(uint8_t *wbuf, const uint8_t *src, int bytes, uint64_t *bar) {
  fence_proxy_async();
  mbar_expect_tx(bar, (uint32_t)bytes);
  bulk_g2s(wbuf, src, (uint32_t)bytes, bar);
}

// ---- the arithmetic: mma.sync.m16n8k16 -----------------------------------------------------------------------
// A 16-weight scale group of Q6_K is exactly one k-step of the MMA. A = the codes as exact fp16 integers q - 32
// (byte under the exponent 0x64 = 1024 + q, minus 1056), B = the activations as two fp16 planes (x * s = hi + lo,
// s a power of two per activation row that puts its largest magnitude in [2^13, 2^14); the planes are adjacent
// columns, four rows per MMA), C starts at zero every k-step and enters the superblock's sum through one f32 FMA
// with the group's int8 scale; d is applied once per superblock, 1 / s at the end. Within a group the MMA's k index
// is permuted so that lane t of a fragment row owns four consecutive codes (one 32-bit word of low nibbles, one of
// high bit pairs): MMA columns (2t, 2t+1, 2t+8, 2t+9) stand for weights 4t .. 4t+3, on both operands.
//
// Shared memory of a caller (Bufs): one or two weight-block buffers, the pass's f32 activation rows, the
// B fragments of every k-step ([K/16][2][32] x 8 bytes, built once per expert and token pass and used by every
// row block of the expert), the partial sums of the warps that share a 16-row tile ([4 tiles][WARPS/4][2][2][32]
// f32), the kTok inverse scales and scales, two mbarriers for the blocks' bulk copies.
__host__ __device__ inline size_t block_bytes(int K) { return ((size_t)kRows * (K / KNJ_QK_K) * KNJ_Q6K_BYTES + 15) & ~(size_t)15; }
__host__ __device__ inline size_t panel_bytes(int K) { return (size_t)(K / 16) * 2 * 32 * 8; }
__host__ __device__ inline size_t red_bytes(int warps) { return (size_t)4 * (warps / 4) * 2 * 2 * 32 * 4; }
// bytes behind the weight-block buffer(s): the pass's activation rows, panel, partial sums, scales
__host__ __device__ inline size_t act_scratch_bytes(int K, int warps) {
  return (size_t)kTok * K * 4 + panel_bytes(K) + red_bytes(warps) + 2 * kTok * 4;
}

struct Bufs {
  uint8_t *w[2];   // weight blocks (w[1] == w[0]: no double buffering)
  float *abuf;     // [kTok][K] f32: the pass's activation rows
  uint2 *panel;
  float *red, *inv;
  uint64_t *bars;  // [2], initialised by the caller with one arrival each
  int *fail;       // shared flag a wait that gives up raises
};
__device__ __forceinline__ Bufs carve(uint8_t *base, int K, int warps, bool two_blocks, uint64_t *bars, int *fail) {
  Bufs b;
  b.w[0] = base;
  b.w[1] = two_blocks ? base + block_bytes(K) : base;
  uint8_t *p = base + (two_blocks ? 2 : 1) * block_bytes(K);
  b.abuf = reinterpret_cast<float *>(p);
  b.panel = reinterpret_cast<uint2 *>(p + (size_t)kTok * K * 4);
  b.red = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(b.panel) + panel_bytes(K));
  b.inv = b.red + red_bytes(warps) / 4;
  b.bars = bars;
  b.fail = fail;
  return b;
}

// 32 bits from a 2-byte aligned shared-memory address (the same alignment for every lane of the warp)
__device__ __forceinline__ uint32_t lds32_u16(const uint8_t *p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
  return (a & 2) ? __byte_perm(q[0], q[1], 0x5432) : q[0];
}

// Scales and B fragments of the nt activation rows staged at b.abuf. Every thread of the CTA; ends with a CTA barrier.
template <int WARPS>
__device__ __forceinline__ void prepare_panel(const Bufs &b, int K, int nt, int lane, int warp) {
  const int tid = warp * 32 + lane, ksteps = K / 16, NG = nt > 4 ? 2 : 1;
  float *inv = b.inv, *scl = b.inv + kTok;
  for (int t = warp; t < nt; t += WARPS) {
    const float4 *x = reinterpret_cast<const float4 *>(b.abuf + (size_t)t * K);
    float amax = 0.f;
    for (int i = lane; i < K / 4; i += 32) {
      const float4 v = x[i];
      amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) {
      const int ex = (amax > 0.f && amax < 3.0e38f) ? ilogbf(amax) : 13;
      scl[t] = ldexpf(1.0f, 13 - ex);
      inv[t] = ldexpf(1.0f, ex - 13);
    }
  }
  __syncthreads();
  // entry (k-step s, group q, lane (g, t)) = activations 16 s + 4 t .. + 3 of row 4 q + g / 2, plane g % 2
  for (int i = tid; i < ksteps * NG * 32; i += WARPS * 32) {
    const int ln = i & 31, q = NG == 2 ? (i >> 5) & 1 : 0, s_ = NG == 2 ? i >> 6 : i >> 5;
    const int g = ln >> 2, t = ln & 3, row = 4 * q + (g >> 1);
    uint2 out = make_uint2(0u, 0u);
    if (row < nt) {
      const float4 x = *reinterpret_cast<const float4 *>(b.abuf + (size_t)row * K + 16 * s_ + 4 * t);
      const float sc = scl[row];
      const float v[4] = {x.x * sc, x.y * sc, x.z * sc, x.w * sc};
      __half h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        h[j] = __float2half_rn(v[j]);
        if (g & 1) h[j] = __float2half_rn(v[j] - __half2float(h[j]));
      }
      out.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
      out.y = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
    }
    b.panel[((size_t)s_ * 2 + q) * 32 + ln] = out;
  }
  __syncthreads();
}

// One staged block of up to 64 rows against the prepared panel. warp = (16-row tile, K part); a unit is a quarter
// superblock: the four scale groups (c = 0..3) of (half hf, sixteen-lane half hh) share one word of high bit pairs
// and two words of low nibbles per row. One CTA barrier inside (between the partial sums and their reduction): when
// a thread returns, every warp has finished reading wbuf. The caller puts a CTA barrier before the next call.
template <int NG, int WARPS, class Store>
__device__ __forceinline__ void block_mma(const uint8_t *wbuf, const Bufs &b, int K, int n_rows, int nt, int lane, int warp, Store store) {
  constexpr int S = WARPS / 4;  // warps that share a tile, each with a contiguous part of K
  static_assert(WARPS % 4 == 0 && S >= 1, "four 16-row tiles per block");
  const int tid = warp * 32 + lane, nsb = K / KNJ_QK_K, row_bytes = nsb * KNJ_Q6K_BYTES;
  const uint2 *panel = b.panel;
  float *red = b.red;
  const int tile = warp & 3, part = warp >> 2, n_tiles = (n_rows + 15) >> 4;
  const int g = lane >> 2, t = lane & 3;
  float acc[NG][2];
#pragma unroll
  for (int q = 0; q < NG; ++q) acc[q][0] = acc[q][1] = 0.f;
  if (tile < n_tiles) {
    const int units = 4 * nsb, u0 = units * part / S, u1 = units * (part + 1) / S;
    const uint8_t *r0 = wbuf + (size_t)(16 * tile + g) * row_bytes, *r1 = r0 + 8 * (size_t)row_bytes;
    const __half2 k1056 = __float2half2_rn(1056.0f);
    float psum[NG][2];
    int cur_sb = -1;
    for (int u = u0; u < u1; ++u) {
      const int sb = u >> 2, hf = (u >> 1) & 1, hh = u & 1;
      if (sb != cur_sb) {
        if (cur_sb >= 0) {
          const float d0 = knj_half_bits_to_float(*reinterpret_cast<const uint16_t *>(r0 + cur_sb * KNJ_Q6K_BYTES + 208));
          const float d1 = knj_half_bits_to_float(*reinterpret_cast<const uint16_t *>(r1 + cur_sb * KNJ_Q6K_BYTES + 208));
#pragma unroll
          for (int q = 0; q < NG; ++q) {
            acc[q][0] = fmaf(d0, psum[q][0], acc[q][0]);
            acc[q][1] = fmaf(d1, psum[q][1], acc[q][1]);
          }
        }
        cur_sb = sb;
#pragma unroll
        for (int q = 0; q < NG; ++q) psum[q][0] = psum[q][1] = 0.f;
      }
      const uint8_t *b0 = r0 + sb * KNJ_Q6K_BYTES, *b1 = r1 + sb * KNJ_Q6K_BYTES;
      const int off = 16 * hh + 4 * t;
      const uint32_t qh0 = lds32_u16(b0 + 128 + 32 * hf + off), qh1 = lds32_u16(b1 + 128 + 32 * hf + off);
      const int8_t *sc0 = reinterpret_cast<const int8_t *>(b0) + 192 + 8 * hf + hh;
      const int8_t *sc1 = reinterpret_cast<const int8_t *>(b1) + 192 + 8 * hf + hh;
#pragma unroll
      for (int cp = 0; cp < 2; ++cp) {
        const uint32_t ql0 = lds32_u16(b0 + 64 * hf + 32 * cp + off), ql1 = lds32_u16(b1 + 64 * hf + 32 * cp + off);
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const int c = cp + 2 * ch;
          const uint32_t q0 = ((ql0 >> (4 * ch)) & 0x0f0f0f0fu) | (((qh0 >> (2 * c)) & 0x03030303u) << 4);
          const uint32_t q1 = ((ql1 >> (4 * ch)) & 0x0f0f0f0fu) | (((qh1 >> (2 * c)) & 0x03030303u) << 4);
          const uint32_t e0l = __byte_perm(q0, 0x64646464u, 0x4140), e0h = __byte_perm(q0, 0x64646464u, 0x4342);
          const uint32_t e1l = __byte_perm(q1, 0x64646464u, 0x4140), e1h = __byte_perm(q1, 0x64646464u, 0x4342);
          const __half2 a0 = __hsub2(*reinterpret_cast<const __half2 *>(&e0l), k1056);  // row g,     k = 2t, 2t+1
          const __half2 a1 = __hsub2(*reinterpret_cast<const __half2 *>(&e1l), k1056);  // row g + 8, k = 2t, 2t+1
          const __half2 a2 = __hsub2(*reinterpret_cast<const __half2 *>(&e0h), k1056);  // row g,     k = 2t+8, 2t+9
          const __half2 a3 = __hsub2(*reinterpret_cast<const __half2 *>(&e1h), k1056);  // row g + 8, k = 2t+8, 2t+9
          const float s0 = (float)sc0[2 * c], s1 = (float)sc1[2 * c];
          const int ks = 16 * sb + 8 * hf + 2 * c + hh;
#pragma unroll
          for (int q = 0; q < NG; ++q) {
            const uint2 bf = panel[((size_t)ks * 2 + q) * 32 + lane];
            float cfr[4];
            mma_f16_16816_zero(cfr, *reinterpret_cast<const uint32_t *>(&a0), *reinterpret_cast<const uint32_t *>(&a1),
                               *reinterpret_cast<const uint32_t *>(&a2), *reinterpret_cast<const uint32_t *>(&a3), bf.x, bf.y);
            psum[q][0] = fmaf(s0, cfr[0] + cfr[1], psum[q][0]);
            psum[q][1] = fmaf(s1, cfr[2] + cfr[3], psum[q][1]);
          }
        }
      }
    }
    if (cur_sb >= 0) {
      const float d0 = knj_half_bits_to_float(*reinterpret_cast<const uint16_t *>(r0 + cur_sb * KNJ_Q6K_BYTES + 208));
      const float d1 = knj_half_bits_to_float(*reinterpret_cast<const uint16_t *>(r1 + cur_sb * KNJ_Q6K_BYTES + 208));
#pragma unroll
      for (int q = 0; q < NG; ++q) {
        acc[q][0] = fmaf(d0, psum[q][0], acc[q][0]);
        acc[q][1] = fmaf(d1, psum[q][1], acc[q][1]);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    red[(((size_t)tile * S + part) * 2 + q) * 64 + lane] = acc[q][0];
    red[(((size_t)tile * S + part) * 2 + q) * 64 + 32 + lane] = acc[q][1];
  }
  __syncthreads();
  // the parts of a tile meet in a fixed order; lane (g, t) of group q held rows g and g + 8 of activation row 4 q + t
  for (int i = tid; i < n_rows * nt; i += WARPS * 32) {
    const int r = i / nt, tk = i - r * nt;
    const int tl = r >> 4, r16 = r & 15, ln = 4 * (r16 & 7) + (tk & 3), q = tk >> 2;
    float v = 0.f;
#pragma unroll
    for (int p_ = 0; p_ < S; ++p_) v += red[(((size_t)tl * S + p_) * 2 + q) * 64 + 32 * (r16 >> 3) + ln];
    store(r, tk, v * b.inv[tk]);
  }
}

// One pass of up to kTok activation rows (row t = A + rows_of[t] * K in global memory; rows_of in shared memory)
// over n_rows consecutive weight rows of one expert starting at src (a multiple of 64 rows into the expert's
// matrix), 64 at a time: Y[rows_of[t] * ldy + r] = the sum for weight row r < n_rows. `bulk`: the blocks travel as
// bulk copies, the next one under way while this one is worked on when b holds two buffers; `staged` counts the
// bulk copies this CTA has waited for (buffer = staged & 1, barrier phase = staged >> 1 & 1). Every thread of the
// CTA calls it with the same arguments; the caller puts a CTA barrier between two calls. False: a wait gave up.
template <int WARPS>
__device__ __forceinline__ bool chunk_pass(const Bufs &b, const uint8_t *src, int n_rows, int K, const float *A, float *Y, int ldy,
                                           const int *rows_of, int nt, unsigned &staged, bool bulk, long long wait_cycles, int lane,
                                           int warp) {
  const int tid = warp * 32 + lane, row_bytes = K / KNJ_QK_K * KNJ_Q6K_BYTES;
  const int nsub = (n_rows + kRows - 1) / kRows;
  const bool two = b.w[1] != b.w[0];
  // the first block travels while the activation side is prepared
  if (bulk && tid == 0) stage_block_bulk(b.w[two ? (staged & 1u) : 0], src, min(kRows, n_rows) * row_bytes, &b.bars[staged & 1u]);
  for (int i = tid; i < nt * (K / 4); i += WARPS * 32) {
    const int t = i / (K / 4), k4 = i - t * (K / 4);
    reinterpret_cast<float4 *>(b.abuf + (size_t)t * K)[k4] = __ldcg(reinterpret_cast<const float4 *>(A + (size_t)rows_of[t] * K) + k4);
  }
  __syncthreads();
  prepare_panel<WARPS>(b, K, nt, lane, warp);
  for (int sub = 0; sub < nsub; ++sub) {
    const int r0 = sub * kRows, nr = min(kRows, n_rows - r0);
    const uint8_t *wbuf;
    if (bulk) {
      wbuf = b.w[two ? (staged & 1u) : 0];
      const bool landed = mbar_wait_for(&b.bars[staged & 1u], (staged >> 1) & 1u, wait_cycles, b.fail);
      ++staged;
      // also: every warp is done with the previous block (and with the partial sums of its reduction)
      if (!__syncthreads_and(landed)) return false;
      if (sub + 1 < nsub && two && tid == 0)
        stage_block_bulk(b.w[staged & 1u], src + (size_t)(r0 + kRows) * row_bytes, min(kRows, n_rows - r0 - kRows) * row_bytes,
                         &b.bars[staged & 1u]);
    } else {
      __syncthreads();
      stage_block(b.w[0], src + (size_t)r0 * row_bytes, nr * row_bytes, tid, WARPS * 32);
      __syncthreads();
      wbuf = b.w[0];
    }
    auto store = [&](int r, int t, float v) { Y[(size_t)rows_of[t] * ldy + r0 + r] = v; };
    if (nt <= 4) block_mma<1, WARPS>(wbuf, b, K, nr, nt, lane, warp, store);
    else block_mma<2, WARPS>(wbuf, b, K, nr, nt, lane, warp, store);
    if (bulk && !two && sub + 1 < nsub) {  // one buffer: the next block can only start once this one is done with
      __syncthreads();
      if (tid == 0)
        stage_block_bulk(b.w[0], src + (size_t)(r0 + kRows) * row_bytes, min(kRows, n_rows - r0 - kRows) * row_bytes, &b.bars[staged & 1u]);
    }
  }
  return true;
}

}  // namespace q6b
}  // namespace knj
