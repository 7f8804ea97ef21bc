/* knj_pack.h -- the project's own W4-g128 expert pack, CUDA/host edition.
 *
 * Same constants, names and semantics as the reference kernels/knj_pack.h
 * (group constants :90-113, knj_bytes_per_weight :76, knj_unpack8_u4 :151,
 * knj_act_words_per_8k :163, knj_pack_group_u4 :196, knj_deinterleave8 :208).
 *
 * One group = 128 weights of one output column: 64 payload bytes (weight 2i in
 * the low nibble of byte i, weight 2i+1 in the high nibble), an fp16 scale, a
 * u8 zero point (always 8) and one pad byte = 68 bytes. w = (code - 8) * scale.
 * Activations for the integer-dot kernel are int8, de-interleaved per 8 k into
 * two u32 words: (k0,k2,k4,k6) and (k1,k3,k5,k7).
 */
#ifndef KNJ_PACK_H
#define KNJ_PACK_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define KNJ_PACK_HD __host__ __device__ static inline
#else
#define KNJ_PACK_HD static inline
#endif

#define KNJ_GROUP_EXPERT 128
#define KNJ_GROUP_KV 64
#define KNJ_META_BYTES_PER_GROUP 3

#define KNJ_BITS_PER_WEIGHT_W8 8
#define KNJ_BITS_PER_WEIGHT_W6 6
#define KNJ_BITS_PER_WEIGHT_W4 4
#define KNJ_BITS_PER_WEIGHT_W3 3
#define KNJ_BITS_PER_WEIGHT_W2 2

#define KNJ_W4_BYTES_PER_WEIGHT (0.5f + 3.0f / 128.0f)
#define KNJ_W3_BYTES_PER_WEIGHT (0.375f + 3.0f / 128.0f)
#define KNJ_W2_BYTES_PER_WEIGHT (0.25f + 3.0f / 128.0f)

#define KNJ_W4_PAYLOAD_BYTES(group) (((group) * 4) / 8)
/* payload + fp16 scale + zero point + pad */
#define KNJ_GROUP_STRIDE_BYTES(bits, group) ((((group) * (bits)) / 8) + 4)
#define KNJ_NIBBLE_BIAS 8

KNJ_PACK_HD float knj_bytes_per_weight(int bits, int group) {
  return (float)bits * 0.125f + (float)KNJ_META_BYTES_PER_GROUP / (float)group;
}

/* Eight 4-bit codes in one word -> four even-position codes in the bytes of
 * *lo and four odd-position codes in the bytes of *hi (each 0..15). */
KNJ_PACK_HD void knj_unpack8_u4(uint32_t packed, int *lo, int *hi) {
  const uint32_t mask = 0x0f0f0f0fu;
  *lo = (int)(packed & mask);
  *hi = (int)((packed >> 4) & mask);
}

KNJ_PACK_HD int knj_act_words_per_8k(void) { return 2; }

/* Host-side packers. */
static inline void knj_pack_group_u4(uint8_t *dst, const uint8_t *codes, int group) {
  for (int i = 0; i < group / 2; ++i)
    dst[i] = (uint8_t)((codes[2 * i] & 0x0f) | ((codes[2 * i + 1] & 0x0f) << 4));
}

static inline void knj_deinterleave8(const int8_t *a8, uint32_t *w2) {
  uint32_t ev = 0, od = 0;
  for (int t = 0; t < 4; ++t) {
    ev |= (uint32_t)(uint8_t)a8[2 * t] << (8 * t);
    od |= (uint32_t)(uint8_t)a8[2 * t + 1] << (8 * t);
  }
  w2[0] = ev;
  w2[1] = od;
}

#undef KNJ_PACK_HD
#endif /* KNJ_PACK_H */
