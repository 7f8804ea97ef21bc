// knj_q4k_engine.cuh -- the tile engine of the decode-class expert projections:
// Q4_K weights streamed from HBM once through per-warp TMA rings, multiplied on
// the fp16 tensor cores as EXACT small integers, f32-accurate results.
//
// Arithmetic (the factored form of dot_q4_k, src/loader/dequant.cpp:954-984):
//   y[row][tok] = sum over superblocks of
//                 d * sum_sb sc_sb * sum_k q_k x_k  -  dmin * sum_sb m_sb * sum_k x_k
//   * a 4-bit code q left in place in an fp16 word IS the fp16 subnormal q * 2^-24
//     (q * 2^-20 for a high nibble), so one AND builds two A-fragment elements;
//   * one packed fp16 multiply folds the 6-bit sub-block scale in: q * sc < 1024
//     is still an exact fp16 subnormal, so a whole superblock accumulates inside
//     the tensor core and d is applied once per superblock and row in f32;
//   * activations are split into a high and a low fp16 plane under a power-of-two
//     scale per (token, superblock) -- together ~22 significant bits -- so the
//     products and the f32 accumulation of mma.sync are exact to f32 level;
//   * the min term is one more MMA per superblock: A = the eight 6-bit m_sb,
//     B = the per-32 sums of the token's planes.
//
// Work split. A TEAM of `ks` warps owns a 16-row tile (8 gate + 8 up rows of the
// same output indices, or 16 rows of one matrix); warp `part` of the team owns
// superblock `part` of every row, i.e. the K range [256 part, 256 part + 256).
// The activations of that K range for up to 8 tokens live in the warp's REGISTERS
// as ready-made B fragments for as long as the team stays with one expert, so the
// inner loop reads nothing but weights. Per tile the warps' partial sums meet in
// shared memory (fixed order, one named barrier per tile).
//
// Fragment bookkeeping (m16n8k16, lane = 4 g + t). Lane t of a row owns code
// group t of the superblock: bytes 32t..32t+31 of qs = sub-block 2t in the low
// nibbles and sub-block 2t+1 in the high ones, so it needs only those two scales.
// Word i (bytes 4i..4i+3) feeds one MMA step per nibble kind: bytes 0 and 2 are
// the k pair (2t, 2t+1), bytes 1 and 3 the pair (2t+8, 2t+9). The activation
// planes keep every aligned group of four k in the order (0,2,1,3), so the B
// fragments of step i are 8 consecutive bytes.
#pragma once
#include "knj_common.cuh"
#include "knj_q4k.h"

namespace knj {
namespace q4e {

constexpr int kTileRows = 16;
constexpr int kStageBytes = kTileRows * KNJ_Q4K_BYTES;  // 2304: one superblock column of a 16-row tile
constexpr int kScratchBytes = 1088;                     // per warp: hi plane 512 | lo plane 512 | 8 sums | pad
constexpr int kMaxTok = 8;                              // tokens of one job (the n dimension of the MMA)

__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_h2(__half lo, __half hi) {
  return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

// The activations of one job as B fragments: lane (g, t) holds token g, sub-blocks 2t and 2t+1 of the warp's
// superblock. h/l[2i], h/l[2i+1]: step i of sub-block 2t; [16 + 2i], [17 + 2i]: sub-block 2t+1.
struct BFrag {
  uint32_t h[32], l[32];
  uint32_t sxh, sxl;  // (sum of sub-block 2t, sum of 2t+1) / 64, high and low fp16 plane
  float inv0, inv1;   // 1 / plane scale of tokens 2t and 2t+1 (the columns this lane's accumulators hold)
};

__device__ __forceinline__ void bfrag_clear(BFrag &b) {
#pragma unroll
  for (int i = 0; i < 32; ++i) b.h[i] = b.l[i] = 0u;
  b.sxh = b.sxl = 0u;
  b.inv0 = b.inv1 = 0.f;
}

// One token's 256 values of this warp's superblock -> fp16 planes in the warp's scratch (all lanes take part,
// lane l converts values 8l..8l+7), then the lanes of MMA column `j` (g == j) pick up their fragments.
// Returns nothing; b.inv0 / b.inv1 are set when j is one of this lane's accumulator columns.
__device__ __forceinline__ void bfrag_take_token(BFrag &b, const float (&v)[8], int j, uint8_t *scratch, int lane) {
  const int g = lane >> 2, t = lane & 3;
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = warp_max(amax);
  // power-of-two scale that puts the largest magnitude in [2^13, 2^14)
  const int be = (int)(__float_as_uint(amax) >> 23);
  int e = 0;
  if (amax > 0.f && be != 0xff) e = max(-120, min(120, 140 - be));
  const float s = __uint_as_float((uint32_t)(127 + e) << 23);
  const float inv = __uint_as_float((uint32_t)(127 - e) << 23);
  uint32_t hw[4], lw[4];
  float part = 0.f;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    __half hh[4], ll[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = v[4 * q + i] * s;
      hh[i] = __float2half_rn(f);
      const float hf = __half2float(hh[i]);
      ll[i] = __float2half_rn(f - hf);
      part += hf + __half2float(ll[i]);
    }
    hw[2 * q] = pack_h2(hh[0], hh[2]);
    hw[2 * q + 1] = pack_h2(hh[1], hh[3]);
    lw[2 * q] = pack_h2(ll[0], ll[2]);
    lw[2 * q + 1] = pack_h2(ll[1], ll[3]);
  }
  __syncwarp();  // the previous token's fragments have been read
  *reinterpret_cast<uint4 *>(scratch + 16 * lane) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
  *reinterpret_cast<uint4 *>(scratch + 512 + 16 * lane) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
  part += __shfl_xor_sync(0xffffffffu, part, 1);
  part += __shfl_xor_sync(0xffffffffu, part, 2);
  if ((lane & 3) == 0) reinterpret_cast<float *>(scratch + 1024)[lane >> 2] = part;
  __syncwarp();
  if (g == j) {
    const uint4 *ph = reinterpret_cast<const uint4 *>(scratch + 128 * t);
    const uint4 *pl = reinterpret_cast<const uint4 *>(scratch + 512 + 128 * t);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 a = ph[i], c = pl[i];
      b.h[4 * i] = a.x; b.h[4 * i + 1] = a.y; b.h[4 * i + 2] = a.z; b.h[4 * i + 3] = a.w;
      b.l[4 * i] = c.x; b.l[4 * i + 1] = c.y; b.l[4 * i + 2] = c.z; b.l[4 * i + 3] = c.w;
    }
    const float2 sx = *reinterpret_cast<const float2 *>(scratch + 1024 + 8 * t);
    const float s0 = sx.x * 0.015625f, s1 = sx.y * 0.015625f;  // |sum| < 32 * 2^14: / 64 keeps it inside fp16
    const __half h0 = __float2half_rn(s0), h1 = __float2half_rn(s1);
    b.sxh = pack_h2(h0, h1);
    b.sxl = pack_h2(__float2half_rn(s0 - __half2float(h0)), __float2half_rn(s1 - __half2float(h1)));
  }
  if (j == 2 * t) b.inv0 = inv;
  if (j == 2 * t + 1) b.inv1 = inv;
}

// Eight consecutive activations as f32 (16-byte aligned source).
__device__ __forceinline__ void load8_f32(const void *base, int dtype, int64_t elem, float (&v)[8]) {
  if (dtype == KNJ_DT_F32) {
    const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem);
    const float4 a = __ldcg(p), c = __ldcg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
  } else {
    const uint4 r = __ldcg(reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(base) + elem));
    const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (dtype == KNJ_DT_BF16) {
        v[2 * i] = __uint_as_float(u[i] << 16);
        v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2 *>(&u[i]);
        v[2 * i] = __low2float(h);
        v[2 * i + 1] = __high2float(h);
      }
    }
  }
}

// (sc[2t], sc[2t+1]) and (m[2t], m[2t+1]) of a superblock header as two bytes each (get_scale_min_k4,
// src/loader/dequant.cpp:64-77). sel16 picks halfword (t & 1) of a word, hi_var = (t >= 2).
__device__ __forceinline__ void header_pairs(const uint4 &hd, uint32_t sel16, bool hi_var, uint32_t &sc2, uint32_t &m2) {
  const uint32_t A = __byte_perm(hd.y, 0u, sel16), B = __byte_perm(hd.z, 0u, sel16), C = __byte_perm(hd.w, 0u, sel16);
  const uint32_t sc_lo = A & 0x3f3fu, m_lo = B & 0x3f3fu;
  const uint32_t sc_hi = (C & 0x0f0fu) | ((A >> 2) & 0x3030u);
  const uint32_t m_hi = ((C >> 4) & 0x0f0fu) | ((B >> 2) & 0x3030u);
  sc2 = hi_var ? sc_hi : sc_lo;
  m2 = hi_var ? m_hi : m_lo;
}

// One tile part: the warp's superblock column of a 16-row tile (dense rows of 144 bytes at `stage`) times the
// job's activations. Returns, for this lane's accumulator positions -- (row g, tokens 2t, 2t+1) and
// (row g+8, tokens 2t, 2t+1) -- the superblock's contribution in activation units.
__device__ __forceinline__ float4 tile_part(const uint8_t *stage, const BFrag &b, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const uint8_t *rg = stage + g * KNJ_Q4K_BYTES, *rh = stage + (g + 8) * KNJ_Q4K_BYTES;
  const uint4 hg = *reinterpret_cast<const uint4 *>(rg), hh = *reinterpret_cast<const uint4 *>(rh);
  const uint4 wg0 = *reinterpret_cast<const uint4 *>(rg + KNJ_Q4K_OFF_QS + 32 * t);
  const uint4 wh0 = *reinterpret_cast<const uint4 *>(rh + KNJ_Q4K_OFF_QS + 32 * t);
  const uint4 wg1 = *reinterpret_cast<const uint4 *>(rg + KNJ_Q4K_OFF_QS + 32 * t + 16);
  const uint4 wh1 = *reinterpret_cast<const uint4 *>(rh + KNJ_Q4K_OFF_QS + 32 * t + 16);
  const uint32_t wg[8] = {wg0.x, wg0.y, wg0.z, wg0.w, wg1.x, wg1.y, wg1.z, wg1.w};
  const uint32_t wh[8] = {wh0.x, wh0.y, wh0.z, wh0.w, wh1.x, wh1.y, wh1.z, wh1.w};

  const uint32_t sel16 = (t & 1) ? 0x4432u : 0x4410u;
  uint32_t scg, mg, sch, mh;
  header_pairs(hg, sel16, t >= 2, scg, mg);
  header_pairs(hh, sel16, t >= 2, sch, mh);
  // bytes -> fp16: 0x6400 | n is 1024 + n; the even scale is taken as is, the odd one (high nibbles, which
  // carry a factor 16) divided by 16 -- both exact
  const uint32_t k1024 = 0x64006400u, kSixteenth = 0x2c002c00u, kNeg64 = 0xd400d400u;
  const uint32_t sEg = sub_f16x2(__byte_perm(scg, 0x64646464u, 0x4040u), k1024);
  const uint32_t sOg = fma_f16x2(__byte_perm(scg, 0x64646464u, 0x4141u), kSixteenth, kNeg64);
  const uint32_t sEh = sub_f16x2(__byte_perm(sch, 0x64646464u, 0x4040u), k1024);
  const uint32_t sOh = fma_f16x2(__byte_perm(sch, 0x64646464u, 0x4141u), kSixteenth, kNeg64);
  const uint32_t mmg = sub_f16x2(__byte_perm(mg, 0x64646464u, 0x4140u), k1024);
  const uint32_t mmh = sub_f16x2(__byte_perm(mh, 0x64646464u, 0x4140u), k1024);

  float cm[4], ch[4], cl[4];
  mma_f16_16816_zero(cm, mmg, mmh, mmg, mmh, b.sxh, b.sxl);
#pragma unroll
  for (int i = 0; i < 4; ++i) ch[i] = cl[i] = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t xg = wg[i], xh = wh[i], yg = xg >> 8, yh = xh >> 8;
    {
      const uint32_t a0 = mul_f16x2(xg & 0x000f000fu, sEg), a1 = mul_f16x2(xh & 0x000f000fu, sEh);
      const uint32_t a2 = mul_f16x2(yg & 0x000f000fu, sEg), a3 = mul_f16x2(yh & 0x000f000fu, sEh);
      mma_f16_16816(ch, a0, a1, a2, a3, b.h[2 * i], b.h[2 * i + 1]);
      mma_f16_16816(cl, a0, a1, a2, a3, b.l[2 * i], b.l[2 * i + 1]);
    }
    {
      const uint32_t a0 = mul_f16x2(xg & 0x00f000f0u, sOg), a1 = mul_f16x2(xh & 0x00f000f0u, sOh);
      const uint32_t a2 = mul_f16x2(yg & 0x00f000f0u, sOg), a3 = mul_f16x2(yh & 0x00f000f0u, sOh);
      mma_f16_16816(ch, a0, a1, a2, a3, b.h[16 + 2 * i], b.h[17 + 2 * i]);
      mma_f16_16816(cl, a0, a1, a2, a3, b.l[16 + 2 * i], b.l[17 + 2 * i]);
    }
  }
  // codes carried 2^-24, the sums 1/64
  const float dg = __half2float(__ushort_as_half((unsigned short)(hg.x & 0xffffu))) * 16777216.0f;
  const float ng = __half2float(__ushort_as_half((unsigned short)(hg.x >> 16))) * 64.0f;
  const float dh = __half2float(__ushort_as_half((unsigned short)(hh.x & 0xffffu))) * 16777216.0f;
  const float nh = __half2float(__ushort_as_half((unsigned short)(hh.x >> 16))) * 64.0f;
  float4 r;
  r.x = (dg * (ch[0] + cl[0]) - ng * cm[0]) * b.inv0;
  r.y = (dg * (ch[1] + cl[1]) - ng * cm[1]) * b.inv1;
  r.z = (dh * (ch[2] + cl[2]) - nh * cm[2]) * b.inv0;
  r.w = (dh * (ch[3] + cl[3]) - nh * cm[3]) * b.inv1;
  return r;
}

__device__ __forceinline__ void team_sync(int team, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(threads) : "memory");
}

}  // namespace q4e
}  // namespace knj
