// knj_router.cu -- the stages of the MoE branch around the expert GEMMs, as
// device kernels: RMSNorm, router logits + softmax + exact top-k, the token
// permutation tables, and the ordered weighted combine. In the reference these
// run on the host (src/model/model.cpp:419-460 and :502-507 on the CPU path;
// tools/bench/q4k_stream_ffn.hip:957-1001 and :1305-1313 between the device
// kernels of the benches).
#include "knj_common.cuh"

using namespace knj;

namespace {

// ---------------------------------------------------------------------------
// RMSNorm: one CTA per row. out = (x * scale) * w, the CPU path's operation
// order (src/model/model.cpp:268-269).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rmsnorm_kernel(const void *__restrict__ x, int dtype, int64_t ldx,
                                                      const __nv_bfloat16 *__restrict__ w, float eps, int H,
                                                      float *__restrict__ out) {
  const int r = blockIdx.x;
  __shared__ float red[8];
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    const float v = load_as_f32(x, dtype, (int64_t)r * ldx + i);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float scale = 1.0f / sqrtf(tot / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += 256) {
    const float v = load_as_f32(x, dtype, (int64_t)r * ldx + i);
    out[(size_t)r * H + i] = __fmul_rn(__fmul_rn(v, scale), __bfloat162float(w[i]));
  }
}

// ---------------------------------------------------------------------------
// Router logits: one warp per (expert, chunk of TT tokens). Lane l owns the
// hidden indices 8l + 256i, keeps its slice of the expert row in registers and
// sweeps the tokens of the chunk. f32 accumulate, fixed order (lane partials
// in index order, then a butterfly), so results do not depend on the launch.
// ---------------------------------------------------------------------------
constexpr int kRouterTT = 8;

__global__ void __launch_bounds__(256) router_logits_kernel(const void *__restrict__ x, int dtype, int64_t ldx,
                                                            const __nv_bfloat16 *__restrict__ Wr,
                                                            const float *__restrict__ bias, int T, int H, int E,
                                                            float *__restrict__ logits) {
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int t0 = blockIdx.y * kRouterTT;
  if (e >= E) return;
  float acc[kRouterTT];
#pragma unroll
  for (int tt = 0; tt < kRouterTT; ++tt) acc[tt] = 0.f;
  for (int i = 0; i < H / 256; ++i) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(Wr + (size_t)e * H + 256 * i + 8 * lane));
    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
    float w[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      w[2 * j] = __uint_as_float(u[j] << 16);
      w[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
    }
#pragma unroll
    for (int tt = 0; tt < kRouterTT; ++tt) {
      if (t0 + tt < T) {
        const int64_t base = (int64_t)(t0 + tt) * ldx + 256 * i + 8 * lane;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[tt] = fmaf(w[j], load_as_f32(x, dtype, base + j), acc[tt]);
      }
    }
  }
  const float b = bias ? bias[e] : 0.f;
#pragma unroll
  for (int tt = 0; tt < kRouterTT; ++tt) {
    const float v = warp_sum(acc[tt]);
    if (lane == 0 && t0 + tt < T) logits[(size_t)(t0 + tt) * E + e] = v + b;
  }
}

// ---------------------------------------------------------------------------
// Softmax + exact top-k + renormalise: one warp per token. Selection is by
// (value descending, expert id ascending), the tie rule of the CPU path's
// strict '>' scan (src/model/model.cpp:442-451).
// ---------------------------------------------------------------------------
constexpr int kMaxEPerLane = 8;  // E <= 256

__global__ void __launch_bounds__(128) router_topk_kernel(const float *__restrict__ logits, int T, int E, int k,
                                                          int32_t *__restrict__ pair_exp,
                                                          float *__restrict__ pair_w) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= T) return;
  const int per = (E + 31) / 32;
  float v[kMaxEPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxEPerLane; ++i) {
    const int e = i * 32 + lane;
    v[i] = (i < per && e < E) ? logits[(size_t)t * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float pr[kMaxEPerLane];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxEPerLane; ++i) {
    pr[i] = (v[i] == -INFINITY) ? 0.f : expf(v[i] - mx);
    sum += pr[i];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int i = 0; i < kMaxEPerLane; ++i) pr[i] = pr[i] / sum;

  float keep = 0.f;
  float sel_p[8];
  int sel_e[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    if (s >= k) break;
    // lane-local best, then a butterfly that prefers the larger value and, on
    // equal values, the smaller expert id
    float bv = -INFINITY, bp = 0.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > bv) { bv = v[i]; be = e; bp = pr[i]; }  // ascending e inside a lane: strict '>' keeps the lowest id
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      const float op = __shfl_xor_sync(0xffffffffu, bp, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; bp = op; }
    }
    sel_e[s] = be;
    sel_p[s] = bp;
    keep += bp;
    // retire the winner
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i)
      if (i * 32 + lane == be) v[i] = -INFINITY;
  }
  const float inv = keep > 0.f ? 1.0f / keep : 0.f;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s >= k) break;
      pair_exp[(size_t)t * k + s] = sel_e[s];
      pair_w[(size_t)t * k + s] = sel_p[s] * inv;
    }
  }
}

// ---------------------------------------------------------------------------
// Permutation tables: one CTA per expert walks all pairs in order and compacts
// the ones routed to it (ascending pair id, the order the CPU path's
// ex_tokens_ lists have), then pads its row with -1.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) permute_kernel(const int32_t *__restrict__ pair_exp, int P, int idx_stride,
                                                      int32_t *__restrict__ pair_idx,
                                                      int32_t *__restrict__ pair_cnt) {
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __shared__ int wsum[8];
  __shared__ int base_s;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  int32_t *row = pair_idx + (size_t)e * idx_stride;
  for (int p0 = 0; p0 < P; p0 += 256) {
    const int p = p0 + threadIdx.x;
    const bool hit = p < P && pair_exp[p] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) wsum[warp] = __popc(m);
    __syncthreads();
    int off = base_s;
    for (int w = 0; w < warp; ++w) off += wsum[w];
    const int rank = off + __popc(m & ((1u << lane) - 1u));
    if (hit && rank < idx_stride) row[rank] = p;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < 8; ++w) tot += wsum[w];
      base_s += tot;
    }
    __syncthreads();
  }
  const int cnt = min(base_s, idx_stride);
  for (int i = cnt + threadIdx.x; i < idx_stride; i += 256) row[i] = -1;
  if (threadIdx.x == 0) pair_cnt[e] = cnt;
}

// experts with work, ascending; n_active[0] = how many, n_active[1] = largest count
__global__ void __launch_bounds__(256) active_list_kernel(const int32_t *__restrict__ pair_cnt, int E,
                                                          int32_t *__restrict__ exp_list,
                                                          int32_t *__restrict__ n_active) {
  __shared__ int wsum[8];
  __shared__ int wmax[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int base = 0, mx = 0;
  for (int e0 = 0; e0 < E; e0 += 256) {
    const int e = e0 + threadIdx.x;
    const int c = e < E ? pair_cnt[e] : 0;
    const unsigned m = __ballot_sync(0xffffffffu, c > 0);
    int cm = c;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cm = max(cm, __shfl_xor_sync(0xffffffffu, cm, o));
    if (lane == 0) { wsum[warp] = __popc(m); wmax[warp] = cm; }
    __syncthreads();
    int off = base;
    for (int w = 0; w < warp; ++w) off += wsum[w];
    if (c > 0) exp_list[off + __popc(m & ((1u << lane) - 1u))] = e;
    for (int w = 0; w < 8; ++w) { base += wsum[w]; mx = max(mx, wmax[w]); }
    __syncthreads();
  }
  for (int i = base + threadIdx.x; i < E; i += 256) exp_list[i] = -1;
  if (threadIdx.x == 0) { n_active[0] = base; n_active[1] = mx; }
}

// ---------------------------------------------------------------------------
// Combine: out[t] = resid[t] + sum_s w * Y[row], contributions added in
// ascending expert id starting from zero with separately rounded multiply and
// add -- the CPU path's `dst[i] += wt * src[i]` over its ascending expert loop
// (src/model/model.cpp:464-508). The residual is added last, as the caller of
// the MoE branch does (src/model/model.cpp:652).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ Y, const int32_t *__restrict__ pair_row,
                                                      const int32_t *__restrict__ pair_exp,
                                                      const float *__restrict__ pair_w, const void *__restrict__ resid,
                                                      int resid_dtype, int64_t ld_resid, void *__restrict__ out,
                                                      int out_dtype, int64_t ldo, int H, int k) {
  const int t = blockIdx.x;
  __shared__ int s_row[8];
  __shared__ float s_w[8];
  if (threadIdx.x == 0) {
    int ex[8], ord[8];
    for (int s = 0; s < k; ++s) { ex[s] = pair_exp[(size_t)t * k + s]; ord[s] = s; }
    for (int a = 1; a < k; ++a) {  // insertion sort by expert id
      const int o = ord[a];
      int b = a - 1;
      while (b >= 0 && ex[ord[b]] > ex[o]) { ord[b + 1] = ord[b]; --b; }
      ord[b + 1] = o;
    }
    for (int s = 0; s < k; ++s) {
      const int p = t * k + ord[s];
      s_row[s] = pair_row ? pair_row[p] : p;
      s_w[s] = pair_w[p];
    }
  }
  __syncthreads();
  for (int h = threadIdx.x * 4; h < H; h += 1024) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < k; ++s) {
      const float4 y = __ldg(reinterpret_cast<const float4 *>(Y + (size_t)s_row[s] * H + h));
      const float w = s_w[s];
      acc.x = __fadd_rn(acc.x, __fmul_rn(w, y.x));
      acc.y = __fadd_rn(acc.y, __fmul_rn(w, y.y));
      acc.z = __fadd_rn(acc.z, __fmul_rn(w, y.z));
      acc.w = __fadd_rn(acc.w, __fmul_rn(w, y.w));
    }
    float r[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = r[i];
      if (resid) v = __fadd_rn(load_as_f32(resid, resid_dtype, (int64_t)t * ld_resid + h + i), v);
      store_from_f32(out, out_dtype, (int64_t)t * ldo + h + i, v);
    }
  }
}

__global__ void silu_mul_kernel(const float *__restrict__ G, const float *__restrict__ U, void *__restrict__ A,
                                int a_dtype, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float g = G[i];
    store_from_f32(A, a_dtype, i, (g / (1.0f + expf(-g))) * U[i]);
  }
}

}  // namespace

extern "C" {

int knj_rmsnorm_launch(const void *x, int x_dtype, int64_t ldx, const uint16_t *w_bf16, float eps, int T, int H,
                       float *out, knj_stream_t s) {
  KNJ_REQUIRE(x && w_bf16 && out, "knj_rmsnorm: null pointer");
  KNJ_REQUIRE(H > 0 && x_dtype >= KNJ_DT_F32 && x_dtype <= KNJ_DT_F16, "knj_rmsnorm: bad H / dtype");
  if (T <= 0) return KNJ_OK;
  rmsnorm_kernel<<<T, 256, 0, as_stream(s)>>>(x, x_dtype, ldx, reinterpret_cast<const __nv_bfloat16 *>(w_bf16), eps, H,
                                              out);
  return launch_status("rmsnorm_kernel");
}

int knj_router_topk_launch(const void *x, int x_dtype, int64_t ldx, const uint16_t *Wr_bf16, const float *bias, int T,
                           int H, int E, int k, float *logits, int32_t *pair_exp, float *pair_w, knj_stream_t s) {
  KNJ_REQUIRE(x && Wr_bf16 && logits && pair_exp && pair_w, "knj_router_topk: null pointer");
  KNJ_REQUIRE(H > 0 && H % 256 == 0, "knj_router_topk: H=%d must be a multiple of 256", H);
  KNJ_REQUIRE(E >= 1 && E <= 32 * kMaxEPerLane, "knj_router_topk: E=%d out of range (<= %d)", E, 32 * kMaxEPerLane);
  KNJ_REQUIRE(k >= 1 && k <= 8 && k <= E, "knj_router_topk: top_k=%d out of range (1..8, <= E)", k);
  KNJ_REQUIRE(aligned16(Wr_bf16), "knj_router_topk: router weight must be 16-byte aligned");
  if (T <= 0) return KNJ_OK;
  dim3 grid((E + 7) / 8, (T + kRouterTT - 1) / kRouterTT);
  router_logits_kernel<<<grid, 256, 0, as_stream(s)>>>(x, x_dtype, ldx, reinterpret_cast<const __nv_bfloat16 *>(Wr_bf16),
                                                       bias, T, H, E, logits);
  int rc = launch_status("router_logits_kernel");
  if (rc) return rc;
  router_topk_kernel<<<(T + 3) / 4, 128, 0, as_stream(s)>>>(logits, T, E, k, pair_exp, pair_w);
  return launch_status("router_topk_kernel");
}

int knj_moe_permute_launch(const int32_t *pair_exp, int P, int E, int idx_stride, int32_t *pair_idx, int32_t *pair_cnt,
                           int32_t *exp_list, int32_t *n_active, knj_stream_t s) {
  KNJ_REQUIRE(pair_exp && pair_idx && pair_cnt && exp_list && n_active, "knj_moe_permute: null pointer");
  KNJ_REQUIRE(P >= 0 && E >= 1 && idx_stride >= 1, "knj_moe_permute: bad sizes");
  permute_kernel<<<E, 256, 0, as_stream(s)>>>(pair_exp, P, idx_stride, pair_idx, pair_cnt);
  int rc = launch_status("permute_kernel");
  if (rc) return rc;
  active_list_kernel<<<1, 256, 0, as_stream(s)>>>(pair_cnt, E, exp_list, n_active);
  return launch_status("active_list_kernel");
}

int knj_active_list_launch(const int32_t *pair_cnt, int E, int32_t *exp_list, int32_t *n_active, knj_stream_t s) {
  KNJ_REQUIRE(pair_cnt && exp_list && n_active && E >= 1, "knj_active_list: bad arguments");
  active_list_kernel<<<1, 256, 0, as_stream(s)>>>(pair_cnt, E, exp_list, n_active);
  return launch_status("active_list_kernel");
}

int knj_moe_combine_launch(const float *Y, const int32_t *pair_row, const int32_t *pair_exp, const float *pair_w,
                           const void *resid, int resid_dtype, int64_t ld_resid, void *out, int out_dtype, int64_t ldo,
                           int T, int H, int k, knj_stream_t s) {
  KNJ_REQUIRE(Y && pair_exp && pair_w && out, "knj_moe_combine: null pointer");
  KNJ_REQUIRE(H > 0 && H % 4 == 0 && k >= 1 && k <= 8, "knj_moe_combine: H %% 4 == 0 and 1 <= k <= 8 required");
  KNJ_REQUIRE(aligned16(Y), "knj_moe_combine: Y must be 16-byte aligned");
  if (T <= 0) return KNJ_OK;
  combine_kernel<<<T, 256, 0, as_stream(s)>>>(Y, pair_row, pair_exp, pair_w, resid, resid_dtype, ld_resid, out,
                                              out_dtype, ldo, H, k);
  return launch_status("combine_kernel");
}

int knj_fuse_gateup_silu_launch(const float *G, const float *U, void *A, int a_dtype, int64_t n, knj_stream_t s) {
  KNJ_REQUIRE(G && U && A, "knj_fuse_gateup_silu: null pointer");
  KNJ_REQUIRE(a_dtype >= KNJ_DT_F32 && a_dtype <= KNJ_DT_F16, "knj_fuse_gateup_silu: unknown dtype");
  if (n <= 0) return KNJ_OK;
  const int64_t blocks = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  silu_mul_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, as_stream(s)>>>(G, U, A, a_dtype, n);
  return launch_status("silu_mul_kernel");
}

}  // extern "C"
