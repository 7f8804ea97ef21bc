// knj_router.cu -- the stages of the MoE branch around the expert GEMMs, as
// device kernels: RMSNorm, router logits + softmax + exact top-k, the token
// permutation tables, and the ordered weighted combine. In the reference these
// run on the host (src/model/model.cpp:419-460 and :502-507 on the CPU path;
// tools/bench/q4k_stream_ffn.hip:957-1001 and :1305-1313 between the device
// kernels of the benches).
#include "knj_common.cuh"
#include "knj_topk.cuh"

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

// eight consecutive activations starting at element idx (a multiple of 8; rows 16-byte aligned)
__device__ __forceinline__ void load8_as_f32(const void *base, int dtype, int64_t idx, float (&v)[8]) {
  if (dtype == KNJ_DT_F32) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(base) + idx));
    const float4 b = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(base) + idx) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 r = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(base) + idx));
    const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (dtype == KNJ_DT_BF16) {
        v[2 * j] = __uint_as_float(u[j] << 16);
        v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2 *>(&u[j]);
        v[2 * j] = __low2float(h);
        v[2 * j + 1] = __high2float(h);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Router logits for large token counts on the warp-level tensor cores
// (mma.sync m16n8k16, bf16 x bf16 -> f32). A warp owns 16 tokens x 64 experts.
// bf16 rows are used as they are; f32 / f16 rows are split on the fly into
// three bf16 planes (hi + mid + lo = 24 significant bits), so every product is
// exact and only the f32 accumulation order differs from the CPU path.
// Both operands are read with one 16-byte load per two k-steps: lane t of a
// quad takes k = 8t..8t+7 of a 32-wide span for its row, and the same mapping
// is used for the router row, so the k-slots of A and B agree.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// CTA = 4 warps = 64 tokens x 64 experts; K in steps of 32 through a 3-stage
// cp.async pipeline (activation tile + router tile per stage).
template <int DT>
__global__ void __launch_bounds__(128) router_logits_mma_kernel(const void *__restrict__ x, int64_t ldx,
                                                                const __nv_bfloat16 *__restrict__ Wr,
                                                                const float *__restrict__ bias, int T, int H, int E,
                                                                float *__restrict__ logits) {
  constexpr int ES = DT == KNJ_DT_F32 ? 4 : 2;      // bytes per activation
  constexpr int XROW = 32 * ES;                     // bytes per staged activation row
  constexpr int XTILE = 64 * XROW, WTILE = 64 * 64; // bytes per stage
  constexpr int STAGES = 3;
  __shared__ __align__(16) uint8_t sx[STAGES][XTILE];
  __shared__ __align__(16) uint8_t sw[STAGES][WTILE];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tok0 = blockIdx.y * 64, e0 = blockIdx.x * 64;
  const int nk = H / 32;

  auto issue = [&](int kstep, int st) {
    const int k0 = kstep * 32;
    // activations: 64 rows x XROW bytes
#pragma unroll
    for (int c = tid; c < XTILE / 16; c += 128) {
      const int r = c / (XROW / 16), cc = c % (XROW / 16);
      const int tok = tok0 + r;
      const uint8_t *src = static_cast<const uint8_t *>(x) + ((int64_t)min(tok, T - 1) * ldx + k0) * ES + cc * 16;
      cp_async16(&sx[st][r * XROW + cc * 16], src, tok < T);
    }
    // router rows: 64 experts x 64 bytes
#pragma unroll
    for (int c = tid; c < WTILE / 16; c += 128) {
      const int r = c >> 2, cc = c & 3;
      const int e = e0 + r;
      cp_async16(&sw[st][r * 64 + cc * 16], Wr + (size_t)min(e, E - 1) * H + k0 + cc * 8, e < E);
    }
  };

  float acc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;

  issue(0, 0);
  cp_async_commit();
  if (nk > 1) issue(1, 1);
  cp_async_commit();
  for (int ks = 0; ks < nk; ++ks) {
    cp_async_wait<1>();
    __syncthreads();
    if (ks + 2 < nk) issue(ks + 2, (ks + 2) % STAGES);
    cp_async_commit();
    const int st = ks % STAGES;
    // A fragments of rows g and g+8 of this warp's 16 tokens: k = 8t..8t+7 of the 32-wide span
    uint32_t a0[4], a1[4], a2[4], b0[4], b1[4], b2[4];
    auto planes = [&](int row, uint32_t (&p0)[4], uint32_t (&p1)[4], uint32_t (&p2)[4]) {
      const uint8_t *src = &sx[st][(warp * 16 + row) * XROW + 8 * t * ES];
      if (DT == KNJ_DT_BF16) {
        const uint4 r = *reinterpret_cast<const uint4 *>(src);
        p0[0] = r.x; p0[1] = r.y; p0[2] = r.z; p0[3] = r.w;
      } else {
        float v[8];
        if (DT == KNJ_DT_F32) {
          const float4 u0 = *reinterpret_cast<const float4 *>(src), u1 = *reinterpret_cast<const float4 *>(src + 16);
          v[0] = u0.x; v[1] = u0.y; v[2] = u0.z; v[3] = u0.w; v[4] = u1.x; v[5] = u1.y; v[6] = u1.z; v[7] = u1.w;
        } else {
          const uint4 r = *reinterpret_cast<const uint4 *>(src);
          const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __half2 h = *reinterpret_cast<const __half2 *>(&u[j]);
            v[2 * j] = __low2float(h);
            v[2 * j + 1] = __high2float(h);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a = v[2 * j], b = v[2 * j + 1];
          const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
          a -= __low2float(h); b -= __high2float(h);
          const __nv_bfloat162 m = __floats2bfloat162_rn(a, b);
          a -= __low2float(m); b -= __high2float(m);
          const __nv_bfloat162 l = __floats2bfloat162_rn(a, b);
          p0[j] = *reinterpret_cast<const uint32_t *>(&h);
          p1[j] = *reinterpret_cast<const uint32_t *>(&m);
          p2[j] = *reinterpret_cast<const uint32_t *>(&l);
        }
      }
    };
    planes(g, a0, a1, a2);
    planes(g + 8, b0, b1, b2);
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const uint4 w = *reinterpret_cast<const uint4 *>(&sw[st][(n * 8 + g) * 64 + 16 * t]);
      mma_bf16_16816(acc[n], a0[0], b0[0], a0[1], b0[1], w.x, w.y);
      mma_bf16_16816(acc[n], a0[2], b0[2], a0[3], b0[3], w.z, w.w);
      if (DT != KNJ_DT_BF16) {
        mma_bf16_16816(acc[n], a1[0], b1[0], a1[1], b1[1], w.x, w.y);
        mma_bf16_16816(acc[n], a1[2], b1[2], a1[3], b1[3], w.z, w.w);
        mma_bf16_16816(acc[n], a2[0], b2[0], a2[1], b2[1], w.x, w.y);
        mma_bf16_16816(acc[n], a2[2], b2[2], a2[3], b2[3], w.z, w.w);
      }
    }
  }
  cp_async_wait<0>();
  const int ra = tok0 + warp * 16 + g, rb = ra + 8;
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    const int e = e0 + n * 8 + 2 * t;
    const float bb0 = (bias && e < E) ? bias[e] : 0.f, bb1 = (bias && e + 1 < E) ? bias[e + 1] : 0.f;
    if (ra < T && e < E) logits[(size_t)ra * E + e] = acc[n][0] + bb0;
    if (ra < T && e + 1 < E) logits[(size_t)ra * E + e + 1] = acc[n][1] + bb1;
    if (rb < T && e < E) logits[(size_t)rb * E + e] = acc[n][2] + bb0;
    if (rb < T && e + 1 < E) logits[(size_t)rb * E + e + 1] = acc[n][3] + bb1;
  }
}

__global__ void __launch_bounds__(128) router_topk_kernel(const float *__restrict__ logits, int T, int E, int k,
                                                          int32_t *__restrict__ pair_exp,
                                                          float *__restrict__ pair_w) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= T) return;
  int sel_e[8];
  float sel_w[8];
  warp_topk(logits + (size_t)t * E, E, k, lane, sel_e, sel_w);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s >= k) break;
      pair_exp[(size_t)t * k + s] = sel_e[s];
      pair_w[(size_t)t * k + s] = sel_w[s];
    }
  }
}

// ---------------------------------------------------------------------------
// Counting-sort form of the permutation tables for long pair lists.
// counts[c][e]: pairs of chunk c (256 consecutive pairs) routed to expert e; after the scan, the number of such
// pairs in earlier chunks. The order inside a chunk is recovered from warp match masks, so every expert's row
// lists its pairs in ascending pair id exactly as permute_kernel does.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) permute_count_kernel(const int32_t *__restrict__ pair_exp, int P, int E,
                                                            int32_t *__restrict__ counts) {
  __shared__ int hist[256];
  hist[threadIdx.x] = 0;
  __syncthreads();
  const int p = blockIdx.x * 256 + threadIdx.x;
  const int e = p < P ? pair_exp[p] : -1;
  const bool valid = e >= 0 && e < E;
  const unsigned peers = __match_any_sync(0xffffffffu, valid ? e : -1 - (int)(threadIdx.x & 31));
  if (valid && (threadIdx.x & 31) == (unsigned)(__ffs(peers) - 1)) atomicAdd(&hist[e], __popc(peers));
  __syncthreads();
  if ((int)threadIdx.x < E) counts[(size_t)blockIdx.x * E + threadIdx.x] = hist[threadIdx.x];
}

__global__ void __launch_bounds__(256) permute_scan_kernel(int32_t *__restrict__ counts, int chunks, int E, int idx_stride,
                                                           int32_t *__restrict__ pair_cnt) {
  const int e = blockIdx.x;
  __shared__ int wsum[8];
  __shared__ int s_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  for (int c0 = 0; c0 < chunks; c0 += 256) {
    const int c = c0 + threadIdx.x;
    const int v = c < chunks ? counts[(size_t)c * E + e] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    int off = s_base, tot = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) off += wsum[w];
      tot += wsum[w];
    }
    if (c < chunks) counts[(size_t)c * E + e] = off + incl - v;
    __syncthreads();
    if (threadIdx.x == 0) s_base += tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) pair_cnt[e] = min(s_base, idx_stride);
}

__global__ void __launch_bounds__(256) permute_scatter_kernel(const int32_t *__restrict__ pair_exp, int P, int E,
                                                              const int32_t *__restrict__ base, int idx_stride,
                                                              int32_t *__restrict__ pair_idx) {
  __shared__ int wcnt[8][256];  // per warp and expert: pairs of that expert in the warp, then in the earlier warps
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 8 * 256; i += 256) (&wcnt[0][0])[i] = 0;
  __syncthreads();
  const int p = blockIdx.x * 256 + threadIdx.x;
  const int e = p < P ? pair_exp[p] : -1;
  const bool valid = e >= 0 && e < E;
  const unsigned peers = __match_any_sync(0xffffffffu, valid ? e : -1 - lane);
  const int in_warp = __popc(peers & ((1u << lane) - 1u));
  if (valid && lane == __ffs(peers) - 1) wcnt[warp][e] = __popc(peers);
  __syncthreads();
  if ((int)threadIdx.x < E) {
    int run = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int c = wcnt[w][threadIdx.x];
      wcnt[w][threadIdx.x] = run;
      run += c;
    }
  }
  __syncthreads();
  if (valid) {
    const int pos = base[(size_t)blockIdx.x * E + e] + wcnt[warp][e] + in_warp;
    if (pos < idx_stride) pair_idx[(size_t)e * idx_stride + pos] = p;
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
  int32_t *row = pair_idx + (size_t)e * idx_stride;
  int base = 0;  // identical in every thread
  // eight consecutive pairs per thread and pass: count, block-wide exclusive scan, write in order
  for (int p0 = 0; p0 < P; p0 += 2048) {
    const int first = p0 + threadIdx.x * 8;
    int v[8];
    if (first + 8 <= P && (P & 3) == 0) {
      const int4 a = __ldg(reinterpret_cast<const int4 *>(pair_exp + first));
      const int4 b = __ldg(reinterpret_cast<const int4 *>(pair_exp + first) + 1);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = first + i < P ? pair_exp[first + i] : -1;
    }
    int c = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) c += (v[i] == e);
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    int off = base, tot = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) off += wsum[w];
      tot += wsum[w];
    }
    int rank = off + incl - c;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v[i] == e) {
        if (rank < idx_stride) row[rank] = first + i;
        ++rank;
      }
    base += tot;
    __syncthreads();
  }
  const int cnt = min(base, idx_stride);
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
template <int RDT, int ODT>
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ Y, const int32_t *__restrict__ pair_row,
                                                      const int32_t *__restrict__ pair_exp,
                                                      const float *__restrict__ pair_w, const void *__restrict__ resid,
                                                      int64_t ld_resid, void *__restrict__ out, int64_t ldo, int H,
                                                      int k) {
  const int t = blockIdx.x;
  __shared__ int s_row[8];
  __shared__ float s_w[8];
  __shared__ int s_ex[8];
  __shared__ float s_wraw[8];
  __shared__ int s_rraw[8];
  grid_dep_wait();
  if ((int)threadIdx.x < k) {  // the k slots' metadata in parallel
    const int pp = t * k + threadIdx.x;
    s_ex[threadIdx.x] = pair_exp[pp];
    s_wraw[threadIdx.x] = pair_w[pp];
    s_rraw[threadIdx.x] = pair_row ? pair_row[pp] : pp;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ex[8], ord[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) { ex[s] = s < k ? s_ex[s] : 0x7fffffff; ord[s] = s; }
    for (int a = 1; a < k; ++a) {  // insertion sort by expert id
      const int o = ord[a];
      int b = a - 1;
      while (b >= 0 && ex[ord[b]] > ex[o]) { ord[b + 1] = ord[b]; --b; }
      ord[b + 1] = o;
    }
    for (int s = 0; s < k; ++s) {
      s_row[s] = s_rraw[ord[s]];
      s_w[s] = s_wraw[ord[s]];
    }
  }
  __syncthreads();
  // gridDim.y column slices per token (small batches: more CTAs shorten the chain of dependent loads)
  const int h_per = (H / 4 + gridDim.y - 1) / gridDim.y * 4;
  const int h_lo = blockIdx.y * h_per, h_hi = min(H, h_lo + h_per);
  for (int h = h_lo + threadIdx.x * 4; h < h_hi; h += 1024) {
    float4 y[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (s < k) y[s] = __ldg(reinterpret_cast<const float4 *>(Y + (size_t)s_row[s] * H + h));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < k) {
        const float w = s_w[s];
        acc.x = __fadd_rn(acc.x, __fmul_rn(w, y[s].x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(w, y[s].y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(w, y[s].z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(w, y[s].w));
      }
    }
    float r[4] = {acc.x, acc.y, acc.z, acc.w};
    if (resid) {
#pragma unroll
      for (int i = 0; i < 4; ++i) r[i] = __fadd_rn(load_as_f32(resid, RDT, (int64_t)t * ld_resid + h + i), r[i]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) store_from_f32(out, ODT, (int64_t)t * ldo + h + i, r[i]);
  }
}

// ---------------------------------------------------------------------------
// Decode front end (T <= 64): RMSNorm statistics, router logits, softmax,
// top-k, permutation tables and the prepared activation vectors in ONE launch.
// CTA b computes the logits of expert b for every token (the row's sum of
// squares falls out of the same pass over x) and, if b < T, prepares token b's
// vector; the CTA that finishes last does the per-token top-k and the tables.
// logit = rsqrt(mean(x^2)+eps) * sum_h (Wr[e][h]*wn[h]) * x[h]: the same value as
// the CPU path's router over the normalised row up to f32 summation order.
// ---------------------------------------------------------------------------
struct FrontParams {
  const void *x;
  int x_dtype;
  int64_t ldx;
  const __nv_bfloat16 *norm_w;  // null: no normalisation
  float eps;
  const __nv_bfloat16 *Wr;
  const float *bias;
  int T, H, E, k, idx_stride;
  float *logits;
  int32_t *pair_exp;
  float *pair_w;
  int32_t *pair_idx, *pair_cnt, *exp_list, *n_active;
  float *xn;  // [T][H]: the rows the experts see (normalised where norm_w is given)
  unsigned int *counter;  // [0, 1 + token groups) zero before the launch
#ifdef KNJ_TRACE
  unsigned long long *trace;  // measurement builds, [10]: global-timer stamps of the phases of the CTA that finishes last
#endif
  int tpc;  // tokens per CTA: ceil(T / 8), the logits being a serial walk over a CTA's tokens
};

__device__ __forceinline__ unsigned long long gtime_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

constexpr int kFrontMaxT = 64;
constexpr int kFrontMaxSlices = 8;  // H <= 2048
constexpr int kFrontTok = 8;        // tokens per CTA, at most (FrontParams::tpc is the number in use)

// Grid (ceil(E/8), ceil(T/8)): CTA (eg, tg) computes the logits of experts
// 8eg..8eg+7 (one per warp) for tokens 8tg..8tg+7 and prepares the vectors of
// some of those tokens. The CTA that completes a token group does that group's
// top-k (one warp per token); the CTA that completes the last group builds the
// permutation tables.
template <int DT>
__global__ void __launch_bounds__(256) moe_front_kernel(const FrontParams p) {
  __shared__ float s_scale[kFrontTok];
  __shared__ int s_flag;
  __shared__ int32_t s_pe[kFrontMaxT * 8];
  __shared__ int32_t s_cc[16][256];  // per 32-pair chunk and expert: count, then exclusive base
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int eg = blockIdx.x, tg = blockIdx.y, n_eg = gridDim.x, n_tg = gridDim.y;
  const int nslice = p.H / 256;
  const int e = eg * 8 + warp;
  const int t0 = tg * p.tpc;
#ifdef KNJ_TRACE
  unsigned long long stamp[9];
  stamp[6] = stamp[7] = stamp[8] = 0;
#define KNJ_FRONT_STAMP(i) (stamp[i] = gtime_ns())
#else
#define KNJ_FRONT_STAMP(i) ((void)0)
#endif
  KNJ_FRONT_STAMP(0);

  // ---- logits (and the rows' scales)
  {
    const int ee = e < p.E ? e : p.E - 1;
    float wr[kFrontMaxSlices][8];
#pragma unroll
    for (int i = 0; i < kFrontMaxSlices; ++i) {
      if (i < nslice) {
        load8_as_f32(p.Wr, KNJ_DT_BF16, (int64_t)ee * p.H + 256 * i + 8 * lane, wr[i]);
        if (p.norm_w) {
          float nw[8];
          load8_as_f32(p.norm_w, KNJ_DT_BF16, 256 * i + 8 * lane, nw);
#pragma unroll
          for (int j = 0; j < 8; ++j) wr[i][j] *= nw[j];
        }
      }
    }
    const float bias = (p.bias && e < p.E) ? p.bias[e] : 0.f;
    // the whole row of a token is fetched before it is used and the next token's row
    // travels meanwhile, so a token costs one trip to L2 instead of one per slice
    constexpr int NV = DT == KNJ_DT_F32 ? 2 : 1;  // 16-byte loads per 8 activations
    uint4 ra[kFrontMaxSlices][NV], rb[kFrontMaxSlices][NV];
    auto fetch = [&](int t, uint4 (&r)[kFrontMaxSlices][NV]) {
#pragma unroll
      for (int sl = 0; sl < kFrontMaxSlices; ++sl)
        if (sl < nslice) {
          const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(p.x) +
                                                             ((int64_t)t * p.ldx + 256 * sl + 8 * lane) * (DT == KNJ_DT_F32 ? 4 : 2));
#pragma unroll
          for (int q = 0; q < NV; ++q) r[sl][q] = __ldg(src + q);
        }
    };
    auto unpack = [&](const uint4 (&r)[NV], float (&v)[8]) {
      if (DT == KNJ_DT_F32) {
        v[0] = __uint_as_float(r[0].x); v[1] = __uint_as_float(r[0].y); v[2] = __uint_as_float(r[0].z); v[3] = __uint_as_float(r[0].w);
        v[4] = __uint_as_float(r[NV - 1].x); v[5] = __uint_as_float(r[NV - 1].y); v[6] = __uint_as_float(r[NV - 1].z); v[7] = __uint_as_float(r[NV - 1].w);
      } else {
        const uint32_t u[4] = {r[0].x, r[0].y, r[0].z, r[0].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (DT == KNJ_DT_BF16) {
            v[2 * j] = __uint_as_float(u[j] << 16);
            v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
          } else {
            const __half2 h = *reinterpret_cast<const __half2 *>(&u[j]);
            v[2 * j] = __low2float(h);
            v[2 * j + 1] = __high2float(h);
          }
        }
      }
    };
    auto reduce_store = [&](int i, const uint4 (&r)[kFrontMaxSlices][NV]) {
      float d0 = 0.f, d1 = 0.f, s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int sl = 0; sl < kFrontMaxSlices; ++sl) {
        if (sl < nslice) {
          float v[8];
          unpack(r[sl], v);
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            d0 = fmaf(wr[sl][j], v[j], d0);
            d1 = fmaf(wr[sl][j + 1], v[j + 1], d1);
            s0 = fmaf(v[j], v[j], s0);
            s1 = fmaf(v[j + 1], v[j + 1], s1);
          }
        }
      }
      const float dot = warp_sum(d0 + d1), ss = warp_sum(s0 + s1);
      if (lane == 0) {
        const float scale = p.norm_w ? 1.0f / sqrtf(ss / (float)p.H + p.eps) : 1.0f;
        if (warp == 0) s_scale[i] = scale;
        if (e < p.E) p.logits[(size_t)(t0 + i) * p.E + e] = dot * scale + bias;
      }
    };
    const int nt = min(p.tpc, p.T - t0);
    // the router and norm weights above do not depend on the previous launch and are already on their way;
    // the token rows are the previous layer's output
    grid_dep_wait();
    KNJ_FRONT_STAMP(6);
    if (nt > 0) fetch(t0, ra);
    for (int i = 0; i < nt; i += 2) {
      if (i + 1 < nt) fetch(t0 + i + 1, rb);
      reduce_store(i, ra);
      if (i == 0) KNJ_FRONT_STAMP(7);
      if (i + 1 < nt) {
        if (i + 2 < nt) fetch(t0 + i + 2, ra);
        reduce_store(i + 1, rb);
      }
      if (i == 0) KNJ_FRONT_STAMP(8);
    }
  }
  __syncthreads();
  KNJ_FRONT_STAMP(1);

  // ---- the rows the experts see: CTA (eg, tg) writes tokens t0 + eg, t0 + eg + n_eg, ...
  for (int i = eg; i < p.tpc; i += n_eg) {
    const int t = t0 + i;
    if (t >= p.T) break;
    const float scale = s_scale[i];
    for (int k = threadIdx.x; k < p.H; k += 256) {
      float v = load_as_f32(p.x, DT, (int64_t)t * p.ldx + k);
      if (p.norm_w) v = __fmul_rn(__fmul_rn(v, scale), __bfloat162float(p.norm_w[k]));
      p.xn[(size_t)t * p.H + k] = v;
    }
  }

  // ---- did this CTA complete its token group?
  KNJ_FRONT_STAMP(2);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_flag = (atomicAdd(p.counter + 1 + tg, 1u) == (unsigned)n_eg - 1) ? 1 : 0;
  __syncthreads();
  if (!s_flag) return;
  __threadfence();
  KNJ_FRONT_STAMP(3);

  // ---- top-k of the group's tokens, one warp each
  {
    const int t = t0 + warp;
    if (warp < p.tpc && t < p.T) {
      int sel_e[8];
      float sel_w[8];
      warp_topk(p.logits + (size_t)t * p.E, p.E, p.k, lane, sel_e, sel_w);
      if (lane == 0) {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s >= p.k) break;
          p.pair_exp[(size_t)t * p.k + s] = sel_e[s];
          p.pair_w[(size_t)t * p.k + s] = sel_w[s];
        }
      }
    }
  }

  // ---- did this CTA complete the last group?
  KNJ_FRONT_STAMP(4);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_flag = (atomicAdd(p.counter, 1u) == (unsigned)n_tg - 1) ? 1 : 0;
  __syncthreads();
  if (!s_flag) return;
  __threadfence();
  KNJ_FRONT_STAMP(5);

  // ---- permutation tables. Pairs are taken in chunks of 32 (one per warp pass):
  // count per (chunk, expert), scan over chunks, then every pair knows its rank.
  const int P = p.T * p.k;
  const int n_chunk = (P + 31) / 32;  // <= 16
  for (int i = threadIdx.x; i < P; i += 256) s_pe[i] = __ldcg(p.pair_exp + i);
  for (int i = threadIdx.x; i < n_chunk * 256; i += 256) (&s_cc[0][0])[i] = 0;
  __syncthreads();
  for (int c = warp; c < n_chunk; c += 8) {
    const int q = c * 32 + lane;
    const int pe = q < P ? s_pe[q] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, pe);
    if (pe >= 0 && (peers & ((1u << lane) - 1u)) == 0) s_cc[c][pe] = __popc(peers);  // first lane of each expert
  }
  __syncthreads();
  int cnt = 0;
  if ((int)threadIdx.x < p.E) {
    for (int c = 0; c < n_chunk; ++c) {
      const int n = s_cc[c][threadIdx.x];
      s_cc[c][threadIdx.x] = cnt;
      cnt += n;
    }
  }
  __syncthreads();
  for (int c = warp; c < n_chunk; c += 8) {
    const int q = c * 32 + lane;
    const int pe = q < P ? s_pe[q] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, pe);
    if (pe >= 0) {
      const int rank = s_cc[c][pe] + __popc(peers & ((1u << lane) - 1u));
      if (rank < p.idx_stride) p.pair_idx[(size_t)pe * p.idx_stride + rank] = q;
    }
  }
  if ((int)threadIdx.x < p.E) {
    const int c2 = min(cnt, p.idx_stride);
    for (int i = c2; i < p.idx_stride; ++i) p.pair_idx[(size_t)threadIdx.x * p.idx_stride + i] = -1;
    p.pair_cnt[threadIdx.x] = c2;
    cnt = c2;
  }
  // active experts, ascending
  __shared__ int s_wsum[8], s_wmax[8];
  const unsigned m = __ballot_sync(0xffffffffu, cnt > 0);
  int cm = cnt;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cm = max(cm, __shfl_xor_sync(0xffffffffu, cm, o));
  if (lane == 0) { s_wsum[warp] = __popc(m); s_wmax[warp] = cm; }
  __syncthreads();
  int off = 0, tot = 0, mxc = 0;
  for (int w = 0; w < 8; ++w) {
    if (w < warp) off += s_wsum[w];
    tot += s_wsum[w];
    mxc = max(mxc, s_wmax[w]);
  }
  if (cnt > 0) p.exp_list[off + __popc(m & ((1u << lane) - 1u))] = threadIdx.x;
  for (int i = tot + threadIdx.x; i < p.E; i += 256) p.exp_list[i] = -1;
  if (threadIdx.x == 0) {
    p.n_active[0] = tot;
    p.n_active[1] = mxc;
#ifdef KNJ_TRACE
    if (p.trace) {
      for (int i = 0; i < 6; ++i) p.trace[i] = stamp[i];
      p.trace[6] = gtime_ns();
      p.trace[7] = stamp[6];
      p.trace[8] = stamp[7];
      p.trace[9] = stamp[8];
    }
#endif
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
  int rc;
  if (T >= 32 && H % 32 == 0 && ldx % 8 == 0 && aligned16(x)) {
    dim3 grid((E + 63) / 64, (T + 63) / 64);
    const __nv_bfloat16 *wr = reinterpret_cast<const __nv_bfloat16 *>(Wr_bf16);
    if (x_dtype == KNJ_DT_BF16) router_logits_mma_kernel<KNJ_DT_BF16><<<grid, 128, 0, as_stream(s)>>>(x, ldx, wr, bias, T, H, E, logits);
    else if (x_dtype == KNJ_DT_F32) router_logits_mma_kernel<KNJ_DT_F32><<<grid, 128, 0, as_stream(s)>>>(x, ldx, wr, bias, T, H, E, logits);
    else router_logits_mma_kernel<KNJ_DT_F16><<<grid, 128, 0, as_stream(s)>>>(x, ldx, wr, bias, T, H, E, logits);
    rc = launch_status("router_logits_mma_kernel");
  } else {
    dim3 grid((E + 7) / 8, (T + kRouterTT - 1) / kRouterTT);
    router_logits_kernel<<<grid, 256, 0, as_stream(s)>>>(x, x_dtype, ldx, reinterpret_cast<const __nv_bfloat16 *>(Wr_bf16),
                                                         bias, T, H, E, logits);
    rc = launch_status("router_logits_kernel");
  }
  if (rc) return rc;
  router_topk_kernel<<<(T + 3) / 4, 128, 0, as_stream(s)>>>(logits, T, E, k, pair_exp, pair_w);
  return launch_status("router_topk_kernel");
}

// Large pair lists: the same tables from a three-step counting sort that is parallel over the pairs
// (chunks of 256 pairs: per-chunk expert histogram -> per-expert scan over chunks -> ordered scatter).
size_t knj_moe_permute_scratch_bytes(int P, int E) {
  const size_t chunks = (size_t)(P > 0 ? (P + 255) / 256 : 1);
  return chunks * (size_t)E * sizeof(int32_t);
}

int knj_moe_permute_ws_launch(const int32_t *pair_exp, int P, int E, int idx_stride, int32_t *pair_idx, int32_t *pair_cnt,
                              int32_t *exp_list, int32_t *n_active, void *scratch, size_t scratch_bytes, knj_stream_t s) {
  KNJ_REQUIRE(pair_exp && pair_idx && pair_cnt && exp_list && n_active, "knj_moe_permute_ws: null pointer");
  KNJ_REQUIRE(P >= 0 && E >= 1 && E <= 256 && idx_stride >= 1, "knj_moe_permute_ws: bad sizes (E <= 256)");
  if (P < 8192 || !scratch) return knj_moe_permute_launch(pair_exp, P, E, idx_stride, pair_idx, pair_cnt, exp_list, n_active, s);
  if (scratch_bytes < knj_moe_permute_scratch_bytes(P, E)) {
    set_error("knj_moe_permute_ws: scratch of %zu bytes needed, %zu given", knj_moe_permute_scratch_bytes(P, E), scratch_bytes);
    return KNJ_E_WORKSPACE;
  }
  cudaStream_t st = as_stream(s);
  const int chunks = (P + 255) / 256;
  int32_t *counts = static_cast<int32_t *>(scratch);
  KNJ_CUDA(cudaMemsetAsync(pair_idx, 0xff, (size_t)E * idx_stride * sizeof(int32_t), st));  // -1 padding
  permute_count_kernel<<<chunks, 256, 0, st>>>(pair_exp, P, E, counts);
  int rc = launch_status("permute_count_kernel");
  if (rc) return rc;
  permute_scan_kernel<<<E, 256, 0, st>>>(counts, chunks, E, idx_stride, pair_cnt);
  rc = launch_status("permute_scan_kernel");
  if (rc) return rc;
  permute_scatter_kernel<<<chunks, 256, 0, st>>>(pair_exp, P, E, counts, idx_stride, pair_idx);
  rc = launch_status("permute_scatter_kernel");
  if (rc) return rc;
  active_list_kernel<<<1, 256, 0, st>>>(pair_cnt, E, exp_list, n_active);
  return launch_status("active_list_kernel");
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

#ifdef KNJ_TRACE
static unsigned long long *g_front_trace = nullptr;
// measurement builds only: device buffer of 16 u64 that receives global-timer stamps of the front kernel's phases
void knj_trace_front(void *dev_buf) { g_front_trace = static_cast<unsigned long long *>(dev_buf); }
#endif

int knj_moe_front_launch(const void *x, int x_dtype, int64_t ldx, const uint16_t *norm_w, float eps,
                         const uint16_t *Wr_bf16, const float *bias, int T, int H, int E, int k, float *logits,
                         int32_t *pair_exp, float *pair_w, int32_t *pair_idx, int idx_stride, int32_t *pair_cnt,
                         int32_t *exp_list, int32_t *n_active, float *xn, uint32_t *counter, knj_stream_t s) {
  KNJ_REQUIRE(x && Wr_bf16 && logits && pair_exp && pair_w && pair_idx && pair_cnt && exp_list && n_active && xn && counter,
              "knj_moe_front: null pointer");
  KNJ_REQUIRE(T >= 1 && T <= kFrontMaxT, "knj_moe_front: T=%d out of range (1..%d)", T, kFrontMaxT);
  KNJ_REQUIRE(H % 256 == 0 && H <= 256 * kFrontMaxSlices, "knj_moe_front: H=%d must be a multiple of 256, <= %d", H,
              256 * kFrontMaxSlices);
  KNJ_REQUIRE(E >= 1 && E <= 256 && k >= 1 && k <= 8 && k <= E && idx_stride >= T, "knj_moe_front: bad E / k / stride");
  KNJ_REQUIRE(aligned16(Wr_bf16) && aligned16(xn) && (!norm_w || aligned16(norm_w)) && aligned16(x) && ldx % 8 == 0,
              "knj_moe_front: 16-byte alignment of x rows, weights and normalised rows");
  FrontParams p{};
  p.x = x; p.x_dtype = x_dtype; p.ldx = ldx; p.norm_w = reinterpret_cast<const __nv_bfloat16 *>(norm_w); p.eps = eps;
  p.Wr = reinterpret_cast<const __nv_bfloat16 *>(Wr_bf16); p.bias = bias; p.T = T; p.H = H; p.E = E; p.k = k;
  p.idx_stride = idx_stride; p.logits = logits; p.pair_exp = pair_exp; p.pair_w = pair_w; p.pair_idx = pair_idx;
  p.pair_cnt = pair_cnt; p.exp_list = exp_list; p.n_active = n_active; p.xn = xn;
  p.counter = counter;
#ifdef KNJ_TRACE
  p.trace = g_front_trace;
#endif
  p.tpc = (T + 7) / 8;  // eight token groups at most: ~128 CTAs at every batch, and the serial walk over a CTA's tokens stays short
  const int n_tg = (T + p.tpc - 1) / p.tpc;
  KNJ_CUDA(cudaMemsetAsync(counter, 0, sizeof(uint32_t) * (1 + n_tg), as_stream(s)));
  dim3 grid((E + 7) / 8, n_tg);
  cudaError_t le;
  if (x_dtype == KNJ_DT_F32) le = launch_chain(moe_front_kernel<KNJ_DT_F32>, grid, dim3(256), 0, as_stream(s), p);
  else if (x_dtype == KNJ_DT_BF16) le = launch_chain(moe_front_kernel<KNJ_DT_BF16>, grid, dim3(256), 0, as_stream(s), p);
  else le = launch_chain(moe_front_kernel<KNJ_DT_F16>, grid, dim3(256), 0, as_stream(s), p);
  KNJ_CUDA(le);
  return launch_status("moe_front_kernel");
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
  KNJ_REQUIRE(out_dtype == KNJ_DT_F32 || out_dtype == KNJ_DT_BF16, "knj_moe_combine: out must be f32 or bf16");
  KNJ_REQUIRE(!resid || (resid_dtype >= KNJ_DT_F32 && resid_dtype <= KNJ_DT_F16), "knj_moe_combine: unknown residual dtype");
  cudaStream_t st = as_stream(s);
#define KNJ_COMBINE(R, O) \
  KNJ_CUDA(launch_chain(combine_kernel<R, O>, dim3(T, slices), dim3(256), 0, st, Y, pair_row, pair_exp, pair_w, resid, ld_resid, out, ldo, H, k))
  const int rd = resid ? resid_dtype : KNJ_DT_F32;
  // few tokens: split every row over column slices of at least 256 so that the grid has ~64 CTAs
  int slices = 1;
  while (slices < 8 && T * slices < 64 && H / (slices * 2) >= 256) slices *= 2;
  if (out_dtype == KNJ_DT_F32) {
    if (rd == KNJ_DT_F32) KNJ_COMBINE(KNJ_DT_F32, KNJ_DT_F32);
    else if (rd == KNJ_DT_BF16) KNJ_COMBINE(KNJ_DT_BF16, KNJ_DT_F32);
    else KNJ_COMBINE(KNJ_DT_F16, KNJ_DT_F32);
  } else {
    if (rd == KNJ_DT_F32) KNJ_COMBINE(KNJ_DT_F32, KNJ_DT_BF16);
    else if (rd == KNJ_DT_BF16) KNJ_COMBINE(KNJ_DT_BF16, KNJ_DT_BF16);
    else KNJ_COMBINE(KNJ_DT_F16, KNJ_DT_BF16);
  }
#undef KNJ_COMBINE
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
