// knj_panel.cuh -- layout of the prepared activation vectors ("panels") the
// decode-class projections consume, and the routine that builds one.
//
// Per vector of K values: a power-of-two scale s puts the largest magnitude in
// [2^13, 2^14); x*s is split into a high and a low fp16 plane (x*s = hi + lo to
// ~22 significant bits); every aligned group of four k is stored in the order
// (0,2,1,3) so a 16-byte load yields the tensor-core B fragments of two MMA
// steps; the per-32 sums of hi+lo feed the Q4_K min term. Storage: one
// 1120-byte chunk per 256-wide superblock -- hi plane (512 B), 64 B gap (keeps
// the two planes on disjoint shared-memory banks), lo plane (512 B), eight f32
// sums (32 B) -- then a 16-byte slot holding 1/s.
#pragma once
#include "knj_common.cuh"

namespace knj {

constexpr int kChunkBytes = 1120;
constexpr int kChunkLo = 576;
constexpr int kChunkSx = 1088;

__host__ __device__ inline size_t panel_vec_bytes(int K) { return (size_t)(K / 256) * kChunkBytes + 16; }

#if defined(__CUDACC__)
// Builds one panel vector at `base` from val(k), k in [0, K). Called by all
// threads of a CTA (blockDim.x a multiple of 32, at most 512); `red` is shared
// scratch of at least 16 floats. Contains CTA barriers.
template <class F>
__device__ __forceinline__ void panel_prep_vector(F val, int K, uint8_t *base, float *red) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int nquad = K / 4;
  float amax = 0.f;
  for (int q = tid; q < nquad; q += nthr)
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(val(4 * q + i)));
  amax = warp_max(amax);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int w = 0; w < (nthr >> 5); ++w) amax = fmaxf(amax, red[w]);

  int e = 0;
  if (amax > 0.f && amax < 3.0e38f) {
    int ex;
    frexpf(amax, &ex);  // amax = m * 2^ex, m in [0.5, 1)
    e = max(-120, min(120, 14 - ex));
  }
  const float s = ldexpf(1.0f, e);
  // the quads of one 32-wide sub-block sit in 8 consecutive lanes
  for (int q = tid; q < nquad; q += nthr) {
    float h[4], l[4];
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = val(4 * q + i) * s;
      h[i] = __half2float(__float2half_rn(f));
      l[i] = __half2float(__float2half_rn(f - h[i]));
      part += h[i] + l[i];
    }
    __half2 h01 = __floats2half2_rn(h[0], h[2]), h23 = __floats2half2_rn(h[1], h[3]);
    __half2 l01 = __floats2half2_rn(l[0], l[2]), l23 = __floats2half2_rn(l[1], l[3]);
    uint8_t *chunk = base + (size_t)(q >> 6) * kChunkBytes;
    const int qq = q & 63;
    *reinterpret_cast<uint2 *>(chunk + 8 * qq) =
        make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
    *reinterpret_cast<uint2 *>(chunk + kChunkLo + 8 * qq) =
        make_uint2(*reinterpret_cast<uint32_t *>(&l01), *reinterpret_cast<uint32_t *>(&l23));
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    if ((tid & 7) == 0) reinterpret_cast<float *>(chunk + kChunkSx)[qq >> 3] = part;
    if ((tid & 7) == 1) *reinterpret_cast<uint2 *>(chunk + 512 + 8 * (qq >> 3)) = make_uint2(0u, 0u);  // the gap
  }
  if (tid == 0) {
    float *inv = reinterpret_cast<float *>(base + (size_t)(K / 256) * kChunkBytes);
    inv[0] = ldexpf(1.0f, -e);
    inv[1] = inv[2] = inv[3] = 0.f;
  }
}
#endif

}  // namespace knj
