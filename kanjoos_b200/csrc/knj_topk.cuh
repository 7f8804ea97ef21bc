// knj_topk.cuh -- softmax + exact top-k + renormalise over one token's router
// logits by one warp; shared by the router kernels and the fused decode stack.
#pragma once
#include "knj_common.cuh"

namespace knj {

// ---------------------------------------------------------------------------
// Softmax + exact top-k + renormalise: one warp per token. Selection is by
// (value descending, expert id ascending), the tie rule of the CPU path's
// strict '>' scan (src/model/model.cpp:442-451).
// ---------------------------------------------------------------------------
constexpr int kMaxEPerLane = 8;  // E <= 256

// One warp: softmax over the E logits of a token, exact top-k, renormalised
// weights. Lane 0 ends up holding the k (expert, weight) pairs in sel_e / sel_w.
// EPL = experts per lane the loops cover (E <= 32 * EPL); fewer than the maximum only shortens the loops.
template <int EPL = kMaxEPerLane>
__device__ __forceinline__ void warp_topk(const float *__restrict__ lg, int E, int k, int lane, int (&sel_e)[8],
                                          float (&sel_w)[8]) {
  const int per = (E + 31) / 32;
  float v[EPL], pr[EPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = i * 32 + lane;
    v[i] = (i < per && e < E) ? __ldcg(lg + e) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    pr[i] = (v[i] == -INFINITY) ? 0.f : expf(v[i] - mx);
    sum += pr[i];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int i = 0; i < EPL; ++i) pr[i] = pr[i] / sum;
  // order-preserving integer keys: larger float <=> larger unsigned key
  unsigned key[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const unsigned u = __float_as_uint(v[i]);
    key[i] = (v[i] == -INFINITY) ? 0u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));
  }
  float keep = 0.f;
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    if (s >= k) break;
    // lane-local best (ascending id inside a lane: strict '>' keeps the lowest id), a hardware max over
    // the warp, then the smallest expert id among the lanes that hold that maximum
    unsigned bk = 0u;
    float bp = 0.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (key[i] > bk) { bk = key[i]; be = i * 32 + lane; bp = pr[i]; }
    const unsigned top = __reduce_max_sync(0xffffffffu, bk);
    const int win = __reduce_min_sync(0xffffffffu, (bk == top && bk != 0u) ? be : 0x7fffffff);
    const int src = win & 31;  // expert id = i*32 + lane
    sel_e[s] = win;
    sel_w[s] = __shfl_sync(0xffffffffu, bp, src);
    keep += sel_w[s];
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (i * 32 + lane == win) key[i] = 0u;
  }
  const float inv = keep > 0.f ? 1.0f / keep : 0.f;
#pragma unroll
  for (int s = 0; s < 8; ++s)
    if (s < k) sel_w[s] *= inv;
}

}  // namespace knj
