// knj_stack.cu -- the resident decode stack (RMSNorm -> router -> top-k -> gate/up
// -> SiLU*up -> down -> ordered combine -> residual, layer after layer) for very
// small batches in ONE cooperative launch. The reference runs this loop on the
// host, one stage at a time (src/model/model.cpp:399-510 per layer, the device
// benches tools/bench/q4k_stream_ffn.hip:957-1313 between kernels).
//
// Why: at batch 1 a layer reads 21 MB (3.4 us of HBM time) but a chain of separate
// kernels spends ~40 us on it, all of it dependent launches and round trips. Here
// the whole stack is one grid of one CTA per SM, and the three points per layer at
// which every CTA needs what the others produced (logits -> top-k, activations ->
// down, layer output -> next layer) are grid barriers on a counter in global memory.
//
// Arithmetic: f32 throughout. Logits and RMS statistics repeat moe_front_kernel's
// operation order exactly, so routing decisions are the same bits; the expert
// products are plain f32 dot products in the factored Q4_K form
// (d*sc*sum(q*x) - dmin*m*sum(x) per 32-weight sub-block), combined in ascending
// expert order like combine_kernel.
//
// Work split. Gate/up: the (distinct routed expert, output row) pairs are dealt to
// the CTAs in equal contiguous runs, a warp takes a row pair (gate row n + up row
// n), lane = (superblock, 64-weight quarter). Down: an output column per warp, all
// routed experts' rows of that column in the warp, so the ordered combine and the
// residual add need no further exchange. Weights are read straight from global
// memory with 16-byte loads issued ahead of their use; vectors sit in shared
// memory transposed so that a warp's 16-byte reads are conflict-free.
//
// Every wait is bounded: a barrier that does not complete within ~1 s sets the
// error word, and every CTA that sees it returns.
#include "knj_common.cuh"
#include "knj_q4k.h"
#include "knj_topk.cuh"

#include <vector>

using namespace knj;

namespace {

constexpr int kMaxT = 4;                 // tokens per step
constexpr int kMaxPairs = kMaxT * 8;     // <= one warp's lanes
constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr long long kSpinLimit = 2000000000ll;  // clock cycles, about a second

struct StackLayer {
  const void *x;
  void *out;
  const __nv_bfloat16 *Wr;
  const float *bias;
  const uint8_t *Wg, *Wu, *Wd;
  const __nv_bfloat16 *norm_w;
  int32_t *tap_exp;
  float *tap_w;
  int64_t ldx, ldo;
  float eps;
  int residual, x_dtype, out_dtype;
};

struct StackParams {
  const StackLayer *layers;
  int n_layers, T, H, F, E, k;
  float *logits;       // [T][E]
  float *act;          // [T*k][F]
  unsigned int *sync;  // [0] arrivals, [1] error word; both zero before the launch
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release(unsigned *p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// All CTAs of the grid have arrived `target` times in total. False: a wait ran out (here or elsewhere).
__device__ __forceinline__ bool grid_barrier(unsigned *sync, unsigned target) {
  __syncthreads();
  int ok = 1;
  if (threadIdx.x == 0) {
    __threadfence();
    red_release(sync, 1u);
    const long long t0 = clock64();
    unsigned polls = 0;
    while (ld_acquire(sync) < target) {
      if ((++polls & 63u) == 0u) {
        if (ld_acquire(sync + 1) != 0u) { ok = 0; break; }
        if (clock64() - t0 > kSpinLimit) { atomicExch(sync + 1, 1u); ok = 0; break; }
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

__device__ __forceinline__ uint4 ldcg16(const void *p) { return __ldcg(reinterpret_cast<const uint4 *>(p)); }
__device__ __forceinline__ uint4 ldnc16(const void *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }

__device__ __forceinline__ float ldcg_as_f32(const void *base, int dtype, int64_t i) {
  if (dtype == KNJ_DT_F32) return __ldcg(static_cast<const float *>(base) + i);
  const unsigned short u = __ldcg(static_cast<const unsigned short *>(base) + i);
  return __uint_as_float((unsigned)u << 16);  // bf16
}

// One lane's share of a Q4_K row: the header of its superblock and the 32 code bytes of its quarter.
struct Quarter {
  uint4 hdr, q0, q1;
};
__device__ __forceinline__ void load_quarter(const uint8_t *row, int q, Quarter &w) {
  const uint8_t *sb = row + (size_t)(q >> 2) * KNJ_Q4K_BYTES;
  w.hdr = ldnc16(sb);
  w.q0 = ldnc16(sb + KNJ_Q4K_OFF_QS + 32 * (q & 3));
  w.q1 = ldnc16(sb + KNJ_Q4K_OFF_QS + 32 * (q & 3) + 16);
}

// (d*sc, dmin*m) of sub-blocks 2G and 2G+1 from a superblock header (the 6-bit packing of get_scale_min_k4).
__device__ __forceinline__ void quarter_scales(const uint4 &hdr, int G, float &a0, float &b0, float &a1, float &b1) {
  const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
  const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
  const int sh = 16 * (G & 1);  // bytes 2(G&1), 2(G&1)+1 of a scale word
  unsigned sc, mn;
  if (G < 2) {
    sc = (hdr.y >> sh) & 0x3f3fu;
    mn = (hdr.z >> sh) & 0x3f3fu;
  } else {
    const unsigned hi = (hdr.w >> sh) & 0xffffu;
    sc = (hi & 0x0f0fu) | ((((hdr.y >> sh) & 0xffffu) >> 2) & 0x3030u);
    mn = ((hi >> 4) & 0x0f0fu) | ((((hdr.z >> sh) & 0xffffu) >> 2) & 0x3030u);
  }
  a0 = d * (float)(sc & 0xffu);
  a1 = d * (float)(sc >> 8);
  b0 = dmin * (float)(mn & 0xffu);
  b1 = dmin * (float)(mn >> 8);
}

// byte j of v as an exact float: 0x4B0000vv is 8388608 + vv
template <int J>
__device__ __forceinline__ float byte_f32(unsigned v) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7540u + J)) - 8388608.0f;
}

// sum over the quarter's 64 weights of q * x: S0 for the low nibbles (sub-block 2G), S1 for the high ones.
// xq points at this quarter's first float4 of a transposed vector, consecutive float4s are `stride4` apart.
__device__ __forceinline__ void quarter_dot(const Quarter &w, const float4 *xq, int stride4, float &S0, float &S1) {
  const unsigned words[8] = {w.q0.x, w.q0.y, w.q0.z, w.q0.w, w.q1.x, w.q1.y, w.q1.z, w.q1.w};
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 xl = xq[i * stride4], xh = xq[(8 + i) * stride4];
    const unsigned lo = words[i] & 0x0f0f0f0fu, hi = (words[i] >> 4) & 0x0f0f0f0fu;
    s0 = fmaf(byte_f32<0>(lo), xl.x, s0);
    s0 = fmaf(byte_f32<1>(lo), xl.y, s0);
    s0 = fmaf(byte_f32<2>(lo), xl.z, s0);
    s0 = fmaf(byte_f32<3>(lo), xl.w, s0);
    s1 = fmaf(byte_f32<0>(hi), xh.x, s1);
    s1 = fmaf(byte_f32<1>(hi), xh.y, s1);
    s1 = fmaf(byte_f32<2>(hi), xh.z, s1);
    s1 = fmaf(byte_f32<3>(hi), xh.w, s1);
  }
  S0 = s0;
  S1 = s1;
}
// the same for two rows that share the vector (gate and up)
__device__ __forceinline__ void quarter_dot2(const Quarter &wa, const Quarter &wb, const float4 *xq, int stride4,
                                             float &A0, float &A1, float &B0, float &B1) {
  const unsigned wa8[8] = {wa.q0.x, wa.q0.y, wa.q0.z, wa.q0.w, wa.q1.x, wa.q1.y, wa.q1.z, wa.q1.w};
  const unsigned wb8[8] = {wb.q0.x, wb.q0.y, wb.q0.z, wb.q0.w, wb.q1.x, wb.q1.y, wb.q1.z, wb.q1.w};
  float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 xl = xq[i * stride4], xh = xq[(8 + i) * stride4];
    const unsigned la = wa8[i] & 0x0f0f0f0fu, ha = (wa8[i] >> 4) & 0x0f0f0f0fu;
    const unsigned lb = wb8[i] & 0x0f0f0f0fu, hb = (wb8[i] >> 4) & 0x0f0f0f0fu;
    a0 = fmaf(byte_f32<0>(la), xl.x, a0);
    a0 = fmaf(byte_f32<1>(la), xl.y, a0);
    a0 = fmaf(byte_f32<2>(la), xl.z, a0);
    a0 = fmaf(byte_f32<3>(la), xl.w, a0);
    a1 = fmaf(byte_f32<0>(ha), xh.x, a1);
    a1 = fmaf(byte_f32<1>(ha), xh.y, a1);
    a1 = fmaf(byte_f32<2>(ha), xh.z, a1);
    a1 = fmaf(byte_f32<3>(ha), xh.w, a1);
    b0 = fmaf(byte_f32<0>(lb), xl.x, b0);
    b0 = fmaf(byte_f32<1>(lb), xl.y, b0);
    b0 = fmaf(byte_f32<2>(lb), xl.z, b0);
    b0 = fmaf(byte_f32<3>(lb), xl.w, b0);
    b1 = fmaf(byte_f32<0>(hb), xh.x, b1);
    b1 = fmaf(byte_f32<1>(hb), xh.y, b1);
    b1 = fmaf(byte_f32<2>(hb), xh.z, b1);
    b1 = fmaf(byte_f32<3>(hb), xh.w, b1);
  }
  A0 = a0; A1 = a1; B0 = b0; B1 = b1;
}

// position of element k of a vector with Q quarters in its transposed shared-memory form:
// float4 number (i*Q + q) holds elements 64q + 4i .. 64q + 4i + 3
__device__ __forceinline__ int tpos(int k, int Q) {
  const int q = k >> 6, r = k & 63;
  return (((r >> 2) * Q + q) << 2) + (r & 3);
}

struct Smem {
  float *xs, *xsum, *av, *asum, *ypart;
  int *sel_e, *pair_d, *list, *ord;
  unsigned *dmask;
  float *sel_w, *scale;
  int *n_distinct;
};
__host__ __device__ inline size_t smem_floats(int T, int H, int F, int k) {
  const int P = T * k;
  return (size_t)T * H + (size_t)T * H / 32 + (size_t)P * F + (size_t)P * F / 32 + (size_t)kWarps * P * (F / 64 + 1) +
         (size_t)6 * kMaxPairs + 16;
}
__device__ __forceinline__ Smem carve(float *base, int T, int H, int F, int k) {
  const int P = T * k;
  Smem s;
  s.xs = base;
  s.av = s.xs + (size_t)T * H;
  s.xsum = s.av + (size_t)P * F;
  s.asum = s.xsum + (size_t)T * H / 32;
  s.ypart = s.asum + (size_t)P * F / 32;
  float *r = s.ypart + (size_t)kWarps * P * (F / 64 + 1);
  s.sel_e = reinterpret_cast<int *>(r);
  s.pair_d = s.sel_e + kMaxPairs;
  s.list = s.pair_d + kMaxPairs;
  s.ord = s.list + kMaxPairs;
  s.dmask = reinterpret_cast<unsigned *>(s.ord + kMaxPairs);
  s.sel_w = reinterpret_cast<float *>(s.dmask + kMaxPairs);
  s.scale = s.sel_w + kMaxPairs;
  s.n_distinct = reinterpret_cast<int *>(s.scale + 8);
  return s;
}

__global__ void __launch_bounds__(kThreads, 1) moe_stack_kernel(const StackParams p) {
  extern __shared__ __align__(16) float smem_f[];
  const Smem sm = carve(smem_f, p.T, p.H, p.F, p.k);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int T = p.T, H = p.H, F = p.F, E = p.E, k = p.k, P = T * k;
  const int QH = H / 64, QF = F / 64;  // quarters per row of gate/up and of down
  const int nslice = H / 256;
  const int G = gridDim.x, c = blockIdx.x;
  unsigned arrivals = 0;

  for (int l = 0; l < p.n_layers; ++l) {
    const StackLayer L = p.layers[l];
    const bool xf32 = L.x_dtype == KNJ_DT_F32;

    // ---- row statistics of every token (each CTA for itself) and, in CTA e < E, expert e's logits.
    // Operation order of moe_front_kernel: lane owns elements 256*sl + 8*lane + j, even/odd chains, warp_sum.
    if (warp < T) {
      const int t = warp;
      const bool mine = c < E;
      float d0 = 0.f, d1 = 0.f, s0 = 0.f, s1 = 0.f;
      for (int sl = 0; sl < nslice; ++sl) {
        const int64_t at = (int64_t)t * L.ldx + 256 * sl + 8 * lane;
        float v[8];
        if (xf32) {
          const uint4 r0 = ldcg16(static_cast<const float *>(L.x) + at), r1 = ldcg16(static_cast<const float *>(L.x) + at + 4);
          v[0] = __uint_as_float(r0.x); v[1] = __uint_as_float(r0.y); v[2] = __uint_as_float(r0.z); v[3] = __uint_as_float(r0.w);
          v[4] = __uint_as_float(r1.x); v[5] = __uint_as_float(r1.y); v[6] = __uint_as_float(r1.z); v[7] = __uint_as_float(r1.w);
        } else {
          const uint4 r = ldcg16(static_cast<const unsigned short *>(L.x) + at);
          const unsigned u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[2 * j] = __uint_as_float(u[j] << 16);
            v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
          }
        }
        float wr[8];
        if (mine) {
          const uint4 r = ldnc16(L.Wr + (size_t)c * H + 256 * sl + 8 * lane);
          const unsigned u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            wr[2 * j] = __uint_as_float(u[j] << 16);
            wr[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
          }
          if (L.norm_w) {
            const uint4 rn = ldnc16(L.norm_w + 256 * sl + 8 * lane);
            const unsigned un[4] = {rn.x, rn.y, rn.z, rn.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              wr[2 * j] *= __uint_as_float(un[j] << 16);
              wr[2 * j + 1] *= __uint_as_float(un[j] & 0xffff0000u);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) wr[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          d0 = fmaf(wr[j], v[j], d0);
          d1 = fmaf(wr[j + 1], v[j + 1], d1);
          s0 = fmaf(v[j], v[j], s0);
          s1 = fmaf(v[j + 1], v[j + 1], s1);
        }
      }
      const float dot = warp_sum(d0 + d1), ss = warp_sum(s0 + s1);
      if (lane == 0) {
        const float scale = L.norm_w ? 1.0f / sqrtf(ss / (float)H + L.eps) : 1.0f;
        sm.scale[t] = scale;
        if (mine) {
          const float bias = L.bias ? L.bias[c] : 0.f;
          p.logits[(size_t)t * E + c] = dot * scale + bias;
        }
      }
    }
    __syncthreads();
    // ---- the rows the experts see, transposed in shared memory, and their 32-element sums
    for (int i = threadIdx.x; i < T * H; i += kThreads) {
      const int t = i / H, kx = i - t * H;
      float v = ldcg_as_f32(L.x, L.x_dtype, (int64_t)t * L.ldx + kx);
      if (L.norm_w) v = __fmul_rn(__fmul_rn(v, sm.scale[t]), __bfloat162float(L.norm_w[kx]));
      sm.xs[(size_t)t * H + tpos(kx, QH)] = v;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < T * H / 32; i += kThreads) {
      const int t = i / (H / 32), b = i - t * (H / 32);
      float s = 0.f;
      for (int j = 0; j < 32; ++j) s += sm.xs[(size_t)t * H + tpos(32 * b + j, QH)];
      sm.xsum[i] = s;
    }

    arrivals += G;
    if (!grid_barrier(p.sync, arrivals)) return;

    // ---- top-k per token (every CTA for itself), then the distinct experts in ascending order
    if (warp < T) {
      int se[8];
      float sw[8];
      warp_topk(p.logits + (size_t)warp * E, E, k, lane, se, sw);
      if (lane == 0) {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s >= k) break;
          sm.sel_e[warp * k + s] = se[s];
          sm.sel_w[warp * k + s] = sw[s];
          if (c == 0 && L.tap_exp) L.tap_exp[warp * k + s] = se[s];
          if (c == 0 && L.tap_w) L.tap_w[warp * k + s] = sw[s];
        }
      }
    }
    __syncthreads();
    if (warp == 0) {
      const int e = lane < P ? sm.sel_e[lane] : -1 - lane;  // distinct dummies so that they match nobody
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      const bool first = lane < P && (peers & ((1u << lane) - 1u)) == 0u;
      int d = 0;
      for (int j = 0; j < kMaxPairs; ++j) {
        const int ej = __shfl_sync(0xffffffffu, e, j);
        const int fj = __shfl_sync(0xffffffffu, (int)first, j);
        if (fj && ej < e) ++d;
      }
      if (lane < P) sm.pair_d[lane] = d;
      if (first) {
        sm.list[d] = e;
        sm.dmask[d] = peers;
      }
      const unsigned fm = __ballot_sync(0xffffffffu, first);
      if (lane == 0) *sm.n_distinct = __popc(fm);
      // a token's slots in ascending expert order (the order of the weighted sum)
      if (lane < T) {
        int ex[8], od[8];
        for (int s = 0; s < k; ++s) { ex[s] = sm.sel_e[lane * k + s]; od[s] = s; }
        for (int a = 1; a < k; ++a) {
          const int o = od[a], eo = ex[a];
          int b = a - 1;
          while (b >= 0 && ex[b] > eo) { od[b + 1] = od[b]; ex[b + 1] = ex[b]; --b; }
          od[b + 1] = o;
          ex[b + 1] = eo;
        }
        for (int s = 0; s < k; ++s) sm.ord[lane * k + s] = lane * k + od[s];
      }
    }
    __syncthreads();
    const int D = *sm.n_distinct;

    // ---- gate/up + SiLU*up: row pairs [u0, u1) of this CTA, one per warp at a time
    {
      const long long U = (long long)D * F;
      const int u0 = (int)(U * c / G), u1 = (int)(U * (c + 1) / G);
      const bool live = lane < QH;
      const size_t row_bytes = (size_t)nslice * KNJ_Q4K_BYTES;
      Quarter g0, up0, g1, up1;
      auto fetch = [&](int u, Quarter &wg, Quarter &wu) {
        const int d = u / F, n = u - d * F;
        const size_t row = ((size_t)sm.list[d] * F + n) * row_bytes;
        if (live) {
          load_quarter(L.Wg + row, lane, wg);
          load_quarter(L.Wu + row, lane, wu);
        }
      };
      int u = u0 + warp;
      if (u < u1) fetch(u, g0, up0);
      for (; u < u1; u += kWarps) {
        if (u + kWarps < u1) fetch(u + kWarps, g1, up1);
        const int d = u / F, n = u - d * F;
        float ga0 = 0.f, gb0 = 0.f, ga1 = 0.f, gb1 = 0.f, ua0 = 0.f, ub0 = 0.f, ua1 = 0.f, ub1 = 0.f;
        if (live) {
          quarter_scales(g0.hdr, lane & 3, ga0, gb0, ga1, gb1);
          quarter_scales(up0.hdr, lane & 3, ua0, ub0, ua1, ub1);
        }
        unsigned todo = sm.dmask[d];
        while (todo) {
          const int pr = __ffs(todo) - 1;
          todo &= todo - 1u;
          const int t = pr / k;
          float vg = 0.f, vu = 0.f;
          if (live) {
            float A0, A1, B0, B1;
            quarter_dot2(g0, up0, reinterpret_cast<const float4 *>(sm.xs + (size_t)t * H) + lane, QH, A0, A1, B0, B1);
            const float x0 = sm.xsum[t * (H / 32) + 2 * lane], x1 = sm.xsum[t * (H / 32) + 2 * lane + 1];
            vg = (ga0 * A0 + ga1 * A1) - (gb0 * x0 + gb1 * x1);
            vu = (ua0 * B0 + ua1 * B1) - (ub0 * x0 + ub1 * x1);
          }
          vg = warp_sum(vg);
          vu = warp_sum(vu);
          if (lane == 0) p.act[(size_t)pr * F + n] = (vg / (1.0f + expf(-vg))) * vu;
        }
        g0 = g1;
        up0 = up1;
      }
    }

    // ---- the down rows this warp will need are known already: fetch them before waiting for the activations
    const int n_lo = (int)((long long)H * c / G), n_hi = (int)((long long)H * (c + 1) / G);
    const int tasks = D * QF;              // (distinct expert, quarter) pairs of one output column
    constexpr int kRounds = 3;             // rounds of 32 tasks fetched ahead (8 experts x 12 quarters); later rounds load in place
    const size_t drow_bytes = (size_t)(F / 256) * KNJ_Q4K_BYTES;
    const bool fast = (n_hi - n_lo) <= kWarps;
    Quarter dq[kRounds];
    const int my_col = n_lo + warp;
    if (fast && my_col < n_hi) {
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        const int j = lane + 32 * r;
        if (j < tasks) {
          const int d = j / QF, q = j - d * QF;
          load_quarter(L.Wd + ((size_t)sm.list[d] * H + my_col) * drow_bytes, q, dq[r]);
        }
      }
    }

    arrivals += G;
    if (!grid_barrier(p.sync, arrivals)) return;

    // ---- activations of all pairs, transposed, and their 32-element sums
    for (int i = threadIdx.x; i < P * F; i += kThreads) {
      const int pr = i / F, kx = i - pr * F;
      sm.av[(size_t)pr * F + tpos(kx, QF)] = __ldcg(p.act + i);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < P * F / 32; i += kThreads) {
      const int pr = i / (F / 32), b = i - pr * (F / 32);
      float s = 0.f;
      for (int j = 0; j < 32; ++j) s += sm.av[(size_t)pr * F + tpos(32 * b + j, QF)];
      sm.asum[i] = s;
    }
    __syncthreads();

    // ---- down + ordered combine + residual: one output column per warp
    float *yp = sm.ypart + (size_t)warp * P * (QF + 1);
    for (int n = n_lo + warp; n < n_hi; n += kWarps) {
      for (int r = 0; r * 32 < tasks; ++r) {
        const int j = lane + 32 * r;
        if (j < tasks) {
          const int d = j / QF, q = j - d * QF;
          Quarter w;
          if (fast && n == my_col && r < kRounds) {
            // static indexing keeps dq in registers
            w = dq[0];
#pragma unroll
            for (int rr = 1; rr < kRounds; ++rr)
              if (rr == r) w = dq[rr];
          } else {
            load_quarter(L.Wd + ((size_t)sm.list[d] * H + n) * drow_bytes, q, w);
          }
          float a0, b0, a1, b1;
          quarter_scales(w.hdr, q & 3, a0, b0, a1, b1);
          unsigned todo = sm.dmask[d];
          while (todo) {
            const int pr = __ffs(todo) - 1;
            todo &= todo - 1u;
            float S0, S1;
            quarter_dot(w, reinterpret_cast<const float4 *>(sm.av + (size_t)pr * F) + q, QF, S0, S1);
            const float x0 = sm.asum[pr * (F / 32) + 2 * q], x1 = sm.asum[pr * (F / 32) + 2 * q + 1];
            yp[pr * (QF + 1) + q] = (a0 * S0 + a1 * S1) - (b0 * x0 + b1 * x1);
          }
        }
      }
      __syncwarp();
      if (lane < P) {
        float y = 0.f;
        for (int q = 0; q < QF; ++q) y += yp[lane * (QF + 1) + q];
        yp[lane * (QF + 1) + QF] = y;
      }
      __syncwarp();
      if (lane < T) {
        float acc = 0.f;
        for (int s = 0; s < k; ++s) {
          const int pr = sm.ord[lane * k + s];
          acc = __fadd_rn(acc, __fmul_rn(sm.sel_w[pr], yp[pr * (QF + 1) + QF]));
        }
        if (L.residual) acc = __fadd_rn(ldcg_as_f32(L.x, L.x_dtype, (int64_t)lane * L.ldx + n), acc);
        store_from_f32(L.out, L.out_dtype, (int64_t)lane * L.ldo + n, acc);
      }
      __syncwarp();
    }

    arrivals += G;
    if (l + 1 < p.n_layers && !grid_barrier(p.sync, arrivals)) return;
  }
}

}  // namespace

struct knj_moe_stack {
  StackParams p{};
  void *dev_block = nullptr;  // layer table, logits, activations, sync words
  size_t smem = 0;
  int grid = 0;
  int device = 0;
};

extern "C" {

int knj_moe_stack_create(const knj_moe_ffn_args *layers, int n_layers, knj_moe_stack **out) {
  KNJ_REQUIRE(layers && out && n_layers > 0, "knj_moe_stack_create: null argument or no layers");
  *out = nullptr;
  const knj_moe_ffn_args &a0 = layers[0];
  const int T = a0.n_tokens, H = a0.hidden, F = a0.ffn, E = a0.n_experts, k = a0.top_k;
  KNJ_REQUIRE(T >= 1 && T <= kMaxT, "knj_moe_stack_create: n_tokens=%d, this launch takes 1..%d", T, kMaxT);
  KNJ_REQUIRE(H > 0 && H % 256 == 0 && H <= 2048, "knj_moe_stack_create: hidden=%d must be a multiple of 256, at most 2048", H);
  KNJ_REQUIRE(F > 0 && F % 256 == 0, "knj_moe_stack_create: ffn=%d must be a multiple of 256", F);
  KNJ_REQUIRE(k >= 1 && k <= 8 && k <= E && E <= 256, "knj_moe_stack_create: top_k=%d / n_experts=%d out of range", k, E);
  std::vector<StackLayer> table(n_layers);
  for (int l = 0; l < n_layers; ++l) {
    const knj_moe_ffn_args &a = layers[l];
    KNJ_REQUIRE(a.n_tokens == T && a.hidden == H && a.ffn == F && a.n_experts == E && a.top_k == k,
                "knj_moe_stack_create: layer %d differs in shape from layer 0", l);
    KNJ_REQUIRE(a.x && a.out && a.w_router && a.w_gate && a.w_up && a.w_down, "knj_moe_stack_create: layer %d: null tensor pointer", l);
    KNJ_REQUIRE(a.down_format == 0, "knj_moe_stack_create: layer %d: Q6_K down matrices are not taken by this launch", l);
    KNJ_REQUIRE(a.x_dtype == KNJ_DT_F32 || a.x_dtype == KNJ_DT_BF16, "knj_moe_stack_create: layer %d: x must be f32 or bf16", l);
    KNJ_REQUIRE(a.out_dtype == KNJ_DT_F32 || a.out_dtype == KNJ_DT_BF16, "knj_moe_stack_create: layer %d: out must be f32 or bf16", l);
    KNJ_REQUIRE(a.ldx >= H && a.ldo >= H && a.ldx % 8 == 0, "knj_moe_stack_create: layer %d: bad row strides", l);
    auto al16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    KNJ_REQUIRE(al16(a.x) && al16(a.w_router) && al16(a.w_gate) && al16(a.w_up) && al16(a.w_down) && (!a.norm_w || al16(a.norm_w)),
                "knj_moe_stack_create: layer %d: x, router, norm and expert bases must be 16-byte aligned", l);
    KNJ_REQUIRE(a.x != a.out, "knj_moe_stack_create: layer %d: out must not alias x (other CTAs still read x)", l);
    StackLayer &s = table[l];
    s.x = a.x;
    s.out = a.out;
    s.Wr = reinterpret_cast<const __nv_bfloat16 *>(a.w_router);
    s.bias = a.router_bias;
    s.Wg = a.w_gate;
    s.Wu = a.w_up;
    s.Wd = a.w_down;
    s.norm_w = reinterpret_cast<const __nv_bfloat16 *>(a.norm_w);
    s.tap_exp = a.tap_pair_exp;
    s.tap_w = a.tap_pair_w;
    s.ldx = a.ldx;
    s.ldo = a.ldo;
    s.eps = a.rms_eps;
    s.residual = a.residual;
    s.x_dtype = a.x_dtype;
    s.out_dtype = a.out_dtype;
  }
  knj_moe_stack *st = new knj_moe_stack();
  KNJ_CUDA(cudaGetDevice(&st->device));
  st->smem = smem_floats(T, H, F, k) * sizeof(float);
  cudaDeviceProp prop;
  KNJ_CUDA(cudaGetDeviceProperties(&prop, st->device));
  if (!prop.cooperativeLaunch || st->smem > (size_t)prop.sharedMemPerBlockOptin) {
    set_error("knj_moe_stack_create: the device lacks cooperative launch or %zu bytes of shared memory per block", st->smem);
    delete st;
    return KNJ_E_REFUSE;
  }
  cudaError_t e = cudaFuncSetAttribute(moe_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st->smem);
  int per_sm = 0;
  if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_stack_kernel, kThreads, st->smem);
  if (e != cudaSuccess || per_sm < 1) {
    delete st;
    cudaGetLastError();
    set_error("knj_moe_stack_create: the kernel does not fit an SM (%s)", cudaGetErrorString(e));
    return KNJ_E_RUNTIME;
  }
  st->grid = sm_count();
  const size_t off_logits = ((size_t)n_layers * sizeof(StackLayer) + 255) & ~(size_t)255;
  const size_t off_act = off_logits + (((size_t)T * E * 4 + 255) & ~(size_t)255);
  const size_t off_sync = off_act + (((size_t)T * k * F * 4 + 255) & ~(size_t)255);
  e = cudaMalloc(&st->dev_block, off_sync + 256);
  if (e == cudaSuccess) e = cudaMemcpy(st->dev_block, table.data(), (size_t)n_layers * sizeof(StackLayer), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (st->dev_block) cudaFree(st->dev_block);
    delete st;
    cudaGetLastError();
    set_error("knj_moe_stack_create: device allocation failed (%s)", cudaGetErrorString(e));
    return KNJ_E_RUNTIME;
  }
  char *base = static_cast<char *>(st->dev_block);
  st->p.layers = reinterpret_cast<const StackLayer *>(base);
  st->p.n_layers = n_layers;
  st->p.T = T; st->p.H = H; st->p.F = F; st->p.E = E; st->p.k = k;
  st->p.logits = reinterpret_cast<float *>(base + off_logits);
  st->p.act = reinterpret_cast<float *>(base + off_act);
  st->p.sync = reinterpret_cast<unsigned int *>(base + off_sync);
  *out = st;
  return KNJ_OK;
}

int knj_moe_stack_decode_launch(knj_moe_stack *st, knj_stream_t s) {
  KNJ_REQUIRE(st && st->dev_block, "knj_moe_stack_decode_launch: null stack");
  KNJ_CUDA(cudaMemsetAsync(st->p.sync, 0, 8, as_stream(s)));
  void *args[] = {&st->p};
  KNJ_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(moe_stack_kernel), dim3(st->grid), dim3(kThreads), args,
                                       st->smem, as_stream(s)));
  return launch_status("moe_stack_kernel");
}

int knj_moe_stack_status(knj_moe_stack *st, knj_stream_t s) {
  KNJ_REQUIRE(st && st->dev_block, "knj_moe_stack_status: null stack");
  unsigned int words[2] = {0, 0};
  KNJ_CUDA(cudaMemcpyAsync(words, st->p.sync, 8, cudaMemcpyDeviceToHost, as_stream(s)));
  KNJ_CUDA(cudaStreamSynchronize(as_stream(s)));
  if (words[1] != 0) {
    set_error("knj_moe_stack: a grid barrier ran out of time (arrivals %u)", words[0]);
    return KNJ_E_TIMEOUT;
  }
  return KNJ_OK;
}

void knj_moe_stack_destroy(knj_moe_stack *st) {
  if (!st) return;
  if (st->dev_block) cudaFree(st->dev_block);
  delete st;
}

}  // extern "C"
