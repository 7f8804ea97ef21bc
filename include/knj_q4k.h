/* knj_q4k.h -- GGUF Q4_K / Q6_K superblock decoders, callable from host code
 * and from sm_100a device code.
 *
 * Same names, arguments and results as the reference header
 * kernels/knj_q4k.h (knj_half_bits_to_float :94, knj_load_u16 :121,
 * knj_q4k_scale_min :135, knj_q4k_weight :147, knj_q6k_weight :170,
 * knj_q4k_span16 :215, knj_q6k_span16 :233), written for CUDA: under nvcc the
 * functions are __host__ __device__ and the half conversion compiles to one
 * cvt.f32.f16 on the device, which is exact for every bit pattern.
 *
 * Layouts.
 *   Q4_K  144 B / 256 weights: f16 d @0, f16 dmin @2, 12 B packed 6-bit
 *         scales+mins @4, 128 B codes @16. Sub-block j (32 weights) of code
 *         group g = j/2 uses the low nibbles (j even) or high nibbles (j odd) of
 *         bytes 32g .. 32g+31.  w = (d*sc_j)*q - (dmin*m_j).
 *   Q6_K  210 B / 256 weights: 128 B low nibbles @0, 64 B high 2-bit pairs
 *         @128, 16 int8 scales @192, f16 d @208.  w = d*sc*(q-32).
 */
#ifndef KNJ_Q4K_H
#define KNJ_Q4K_H

#include <stdint.h>
#include <string.h>

#define KNJ_QK_K 256
#define KNJ_Q4K_BYTES 144
#define KNJ_Q6K_BYTES 210

#define KNJ_Q4K_OFF_D 0
#define KNJ_Q4K_OFF_DMIN 2
#define KNJ_Q4K_OFF_SCALE 4
#define KNJ_Q4K_OFF_QS 16

#define KNJ_Q6K_OFF_QL 0
#define KNJ_Q6K_OFF_QH 128
#define KNJ_Q6K_OFF_SC 192
#define KNJ_Q6K_OFF_D 208

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#define KNJ_Q4K_FN __host__ __device__ static inline
#else
#define KNJ_Q4K_FN static inline
#endif

/* IEEE binary16 bits -> binary32, exact (subnormals, infinities, NaN payload). */
KNJ_Q4K_FN float knj_half_bits_to_float(uint16_t h) {
#if defined(__CUDA_ARCH__)
  return __half2float(__ushort_as_half(h));
#else
  const uint32_t sgn = ((uint32_t)h >> 15) << 31;
  uint32_t ex = ((uint32_t)h >> 10) & 0x1fu;
  uint32_t fr = (uint32_t)h & 0x3ffu;
  uint32_t w;
  if (ex == 0x1fu) {
    w = sgn | 0x7f800000u | (fr << 13);
  } else if (ex) {
    w = sgn | ((ex + 112u) << 23) | (fr << 13);
  } else if (!fr) {
    w = sgn;
  } else {
    ex = 113u;
    while (!(fr & 0x400u)) { fr <<= 1; --ex; }
    w = sgn | (ex << 23) | ((fr & 0x3ffu) << 13);
  }
  float f;
  memcpy(&f, &w, sizeof f);
  return f;
#endif
}

/* Little-endian u16 at any byte address (Q6_K metadata is not 2-aligned). */
KNJ_Q4K_FN uint16_t knj_load_u16(const uint8_t *p) {
  return (uint16_t)((uint32_t)p[0] | ((uint32_t)p[1] << 8));
}

/* 6-bit scale *d and min *m of sub-block j (0..7). For j >= 4 the two top
 * bits come from bytes j-4 (scale) and j (min). */
KNJ_Q4K_FN void knj_q4k_scale_min(const uint8_t *scales, int j, uint8_t *d, uint8_t *m) {
  const uint32_t hi = scales[j + 4];
  if (j < 4) {
    *d = (uint8_t)(scales[j] & 0x3fu);
    *m = (uint8_t)(hi & 0x3fu);
  } else {
    *d = (uint8_t)((hi & 0x0fu) | ((uint32_t)(scales[j - 4] >> 6) << 4));
    *m = (uint8_t)((hi >> 4) | ((uint32_t)(scales[j] >> 6) << 4));
  }
}

/* Weight r (0..255) of one Q4_K superblock. */
KNJ_Q4K_FN float knj_q4k_weight(const uint8_t *blk, int r) {
  const int j = r >> 5;
  uint8_t sc, mn;
  knj_q4k_scale_min(blk + KNJ_Q4K_OFF_SCALE, j, &sc, &mn);
  const uint32_t byte = blk[KNJ_Q4K_OFF_QS + ((j >> 1) << 5) + (r & 31)];
  const float q = (float)((byte >> ((j & 1) << 2)) & 0x0fu);
  const float d1 = knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q4K_OFF_D)) * (float)sc;
  const float m1 = knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q4K_OFF_DMIN)) * (float)mn;
  return d1 * q - m1;
}

/* Sixteen consecutive weights r0 .. r0+15 (r0 a multiple of 16, so the span
 * stays inside one sub-block and shares one scale/min). */
KNJ_Q4K_FN void knj_q4k_span16(const uint8_t *blk, int r0, float *out) {
  const int j = r0 >> 5;
  uint8_t sc, mn;
  knj_q4k_scale_min(blk + KNJ_Q4K_OFF_SCALE, j, &sc, &mn);
  const float d1 = knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q4K_OFF_D)) * (float)sc;
  const float m1 = knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q4K_OFF_DMIN)) * (float)mn;
  const uint8_t *q = blk + KNJ_Q4K_OFF_QS + ((j >> 1) << 5) + (r0 & 31);
  const int sh = (j & 1) << 2;
  for (int i = 0; i < 16; ++i) out[i] = d1 * (float)(((uint32_t)q[i] >> sh) & 0x0fu) - m1;
}

/* Weight r (0..255) of one Q6_K superblock. Two 128-weight halves; inside a
 * half, quarter c = (r%128)/32 selects ql[l] (c even) or ql[l+32] (c odd), its
 * low (c < 2) or high nibble, and bits 2c..2c+1 of qh[l]. */
KNJ_Q4K_FN float knj_q6k_weight(const uint8_t *blk, int r) {
  const int hf = r >> 7, c = (r >> 5) & 3, l = r & 31;
  const uint8_t *ql = blk + KNJ_Q6K_OFF_QL + hf * 64;
  const uint8_t *qh = blk + KNJ_Q6K_OFF_QH + hf * 32;
  const int8_t *sc = (const int8_t *)(blk + KNJ_Q6K_OFF_SC) + hf * 8;
  const uint32_t lo = ql[l + ((c & 1) << 5)];
  const uint32_t nib = (c & 2) ? (lo >> 4) : (lo & 0x0fu);
  const uint32_t top = ((uint32_t)qh[l] >> (2 * c)) & 3u;
  const int q = (int)(nib | (top << 4)) - 32;
  const float d = knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q6K_OFF_D));
  return d * (float)sc[(l >> 4) + 2 * c] * (float)q;
}

/* Sixteen consecutive Q6_K weights from r0 (multiple of 16): one int8 scale. */
KNJ_Q4K_FN void knj_q6k_span16(const uint8_t *blk, int r0, float *out) {
  const int hf = r0 >> 7, c = (r0 >> 5) & 3, l = r0 & 31;
  const uint8_t *ql = blk + KNJ_Q6K_OFF_QL + hf * 64 + ((c & 1) << 5) + l;
  const uint8_t *qh = blk + KNJ_Q6K_OFF_QH + hf * 32 + l;
  const int8_t *sc = (const int8_t *)(blk + KNJ_Q6K_OFF_SC) + hf * 8;
  const float s = knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q6K_OFF_D)) * (float)sc[(l >> 4) + 2 * c];
  for (int i = 0; i < 16; ++i) {
    const uint32_t lo = ql[i];
    const uint32_t nib = (c & 2) ? (lo >> 4) : (lo & 0x0fu);
    const uint32_t top = ((uint32_t)qh[i] >> (2 * c)) & 3u;
    out[i] = s * (float)((int)(nib | (top << 4)) - 32);
  }
}

#undef KNJ_Q4K_FN
#endif /* KNJ_Q4K_H */
