/* knj_dot.h -- integer dot-accumulate helpers with the reference's names and
 * semantics (kernels/knj_dot.h: knj_dot4_i32_i8 :117/:130, knj_dot8_i32_i4
 * :149/:155, knj_dot2_i32_i16 :166/:172, capability macros :227-239), over
 * CUDA instead of RDNA inline assembly.
 *
 *   knj_dot4_i32_i8(a, b, acc)   acc + sum_{i<4} s8(a,i) * s8(b,i)      -> dp4a.s32.s32
 *   knj_dot8_i32_i4(a, b, acc)   acc + sum_{i<8} s4(a,i) * s4(b,i), nibble 0 = bits 3..0
 *                                (sm_100a has no 4-bit dot; emulated with shifts)
 *   knj_dot2_i32_i16(a, b, acc)  acc + sum_{i<2} s16(a,i) * s16(b,i)    -> dp2a pair
 *
 * The functions are also callable on the host (plain C arithmetic) so a test
 * can pin the device result to the definition.
 */
#ifndef KNJ_DOT_H
#define KNJ_DOT_H

#include <stdint.h>

#if defined(__CUDACC__)
#define KNJ_DOT_HD __host__ __device__ static inline
#else
#define KNJ_DOT_HD static inline
#endif

KNJ_DOT_HD int knj_dot4_i32_i8(int a, int b, int acc) {
#if defined(__CUDA_ARCH__)
  return __dp4a(a, b, acc);
#else
  for (int i = 0; i < 4; ++i) acc += (int)(int8_t)((uint32_t)a >> (8 * i)) * (int)(int8_t)((uint32_t)b >> (8 * i));
  return acc;
#endif
}

KNJ_DOT_HD int knj_dot8_i32_i4(int a, int b, int acc) {
  for (int i = 0; i < 8; ++i) {
    /* sign-extend nibble i: move it to the top of the word, arithmetic shift back */
    const int x = (int)((uint32_t)a << (28 - 4 * i)) >> 28;
    const int y = (int)((uint32_t)b << (28 - 4 * i)) >> 28;
    acc += x * y;
  }
  return acc;
}

KNJ_DOT_HD int knj_dot2_i32_i16(int a, int b, int acc) {
  const int alo = (int)(int16_t)((uint32_t)a & 0xffffu), ahi = a >> 16;
  const int blo = (int)(int16_t)((uint32_t)b & 0xffffu), bhi = b >> 16;
  return acc + alo * blo + ahi * bhi;
}

#if defined(__cplusplus)
KNJ_DOT_HD int knj_dot4_i32_i8(int a, int b) { return knj_dot4_i32_i8(a, b, 0); }
KNJ_DOT_HD int knj_dot8_i32_i4(int a, int b) { return knj_dot8_i32_i4(a, b, 0); }
KNJ_DOT_HD int knj_dot2_i32_i16(int a, int b) { return knj_dot2_i32_i16(a, b, 0); }
#endif

/* Capability macros keep the reference's names. "ASM" reads as "a native or
 * exactly emulated instruction sequence exists on this target". */
#define KNJ_DOT_ASM_PORTABLE 1
#define KNJ_HAS_DOT4_I8_ASM 1   /* dp4a */
#define KNJ_DOT8_I4_ASM 1       /* emulated, exact */
#define KNJ_DOT2_I16_ASM 1      /* emulated, exact */
#define KNJ_HAS_DOT2_F16_ASM 0  /* no f16 dot-accumulate, as in the reference */
#define KNJ_SDOT4_BUILTIN_PORTABLE 0

#undef KNJ_DOT_HD
#endif /* KNJ_DOT_H */
