// knj_stack_small.cu -- the resident decode stack (RMSNorm -> router -> top-k -> gate/up
// -> SiLU*up -> down -> ordered combine -> residual, layer after layer) for the
// smallest batches (1..4 tokens) in ONE cooperative launch; knj_moe_stack_create
// (knj_stack.cu) picks this kernel for them and the tensor-core form for larger ones. The reference runs this loop on the
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
static_assert(kMaxT * 8 <= 32, "the pairs of a step fit one warp's lanes");
constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr float kUnscale = 0x1p85f;  // undoes the staging scale of the vectors, see word_fma

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
  int slots;           // gate/up row pairs a warp stages at a time (1..3, by the shared memory left)
  long long spin_limit;  // clock cycles a grid barrier may wait
  int stall;             // test hook: added to the first barrier's target, which then cannot complete
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release(unsigned *p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Grid barrier in two halves, so that work that does not depend on the other CTAs can sit between them.
// arrive: everything this CTA wrote so far is published. wait: all CTAs of the grid have arrived `target`
// times in total; false: a wait ran out (here or elsewhere).
__device__ __forceinline__ void grid_arrive(unsigned *sync) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    red_release(sync, 1u);
  }
}
__device__ __forceinline__ bool grid_wait(unsigned *sync, unsigned target, long long limit) {
  int ok = 1;
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    unsigned polls = 0;
    while (ld_acquire(sync) < target) {
      if ((++polls & 63u) == 0u) {
        if (ld_acquire(sync + 1) != 0u) { ok = 0; break; }
        if (clock64() - t0 > limit) { atomicExch(sync + 1, 1u); ok = 0; break; }
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}
__device__ __forceinline__ bool grid_barrier(unsigned *sync, unsigned target, long long limit) {
  grid_arrive(sync);
  return grid_wait(sync, target, limit);
}

// n / dv for the small operands of this kernel (n * dv < 2^32) as one multiply: magic = ceil(2^32 / dv), dv >= 2
__device__ __forceinline__ unsigned div_magic(unsigned dv) { return 0xffffffffu / dv + 1u; }
__device__ __forceinline__ int fast_div(int n, unsigned magic) { return (int)__umulhi((unsigned)n, magic); }

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
  a0 = d * (float)(sc & 0xffu) * kUnscale;
  a1 = d * (float)(sc >> 8) * kUnscale;
  b0 = dmin * (float)(mn & 0xffu);
  b1 = dmin * (float)(mn >> 8);
}

// A code nibble enters the multiply-add WITHOUT a conversion: masked in place at bit p it is the bit pattern of
// the denormal float q * 2^(p-149), which the FMA unit multiplies exactly. The vector element that meets it was
// scaled by 2^(64-p) when it was staged (every element always meets the same nibble position), so each product
// is q * x * 2^-85 and the sums are ordinary normal floats; the factor 2^85 is folded into the block scales.
// Nibbles at bits 20..31 are shifted down by 12 first so that the pattern stays below the exponent field.
// 2^(64-p) for the four elements of a staged float4: low nibbles sit at p = 0, 8, 16, 12 (byte 3 after the
// shift), high nibbles at p = 4, 12, 8, 16 (bytes 2 and 3 after the shift)
__device__ __forceinline__ float4 stage_scale(const float4 &v, bool high) {
  return high ? make_float4(v.x * 0x1p60f, v.y * 0x1p52f, v.z * 0x1p56f, v.w * 0x1p48f)
              : make_float4(v.x * 0x1p64f, v.y * 0x1p56f, v.z * 0x1p48f, v.w * 0x1p52f);
}
__device__ __forceinline__ void word_fma(unsigned w, const float4 &xl, const float4 &xh, float &s0, float &s1) {
  const unsigned v = w >> 12;
  s0 = fmaf(__uint_as_float(w & 0x0000000fu), xl.x, s0);
  s0 = fmaf(__uint_as_float(w & 0x00000f00u), xl.y, s0);
  s0 = fmaf(__uint_as_float(w & 0x000f0000u), xl.z, s0);
  s0 = fmaf(__uint_as_float(v & 0x0000f000u), xl.w, s0);
  s1 = fmaf(__uint_as_float(w & 0x000000f0u), xh.x, s1);
  s1 = fmaf(__uint_as_float(w & 0x0000f000u), xh.y, s1);
  s1 = fmaf(__uint_as_float(v & 0x00000f00u), xh.z, s1);
  s1 = fmaf(__uint_as_float(v & 0x000f0000u), xh.w, s1);
}
// sum over the quarter's 64 weights of q * x: S0 for the low nibbles (sub-block 2G), S1 for the high ones.
// xq points at this quarter's first float4 of a transposed vector, consecutive float4s are `stride4` apart.
// The loops below are deliberately NOT unrolled (two code words per step, the rest of the words rotate down):
// the straight-line form of 64 or 128 weights needs more registers than a 512-thread CTA has and spills.
__device__ __forceinline__ void quarter_dot(const Quarter &w, const float4 *xq, int stride4, float &S0, float &S1) {
  unsigned a0 = w.q0.x, a1 = w.q0.y, a2 = w.q0.z, a3 = w.q0.w, a4 = w.q1.x, a5 = w.q1.y, a6 = w.q1.z, a7 = w.q1.w;
  float s0 = 0.f, s1 = 0.f, t0 = 0.f, t1 = 0.f;
  const float4 *xl = xq, *xh = xq + 8 * stride4;
#pragma unroll 1
  for (int it = 0; it < 4; ++it) {
    const float4 l0 = xl[0], h0 = xh[0], l1 = xl[stride4], h1 = xh[stride4];
    word_fma(a0, l0, h0, s0, s1);
    word_fma(a1, l1, h1, t0, t1);
    a0 = a2; a1 = a3; a2 = a4; a3 = a5; a4 = a6; a5 = a7;
    xl += 2 * stride4;
    xh += 2 * stride4;
  }
  S0 = s0 + t0;
  S1 = s1 + t1;
}
// the same for two rows that share the vector (gate and up)
__device__ __forceinline__ void quarter_dot2(const Quarter &wa, const Quarter &wb, const float4 *xq, int stride4,
                                             float &A0, float &A1, float &B0, float &B1) {
  unsigned a0 = wa.q0.x, a1 = wa.q0.y, a2 = wa.q0.z, a3 = wa.q0.w, a4 = wa.q1.x, a5 = wa.q1.y, a6 = wa.q1.z, a7 = wa.q1.w;
  unsigned b0 = wb.q0.x, b1 = wb.q0.y, b2 = wb.q0.z, b3 = wb.q0.w, b4 = wb.q1.x, b5 = wb.q1.y, b6 = wb.q1.z, b7 = wb.q1.w;
  float sa0 = 0.f, sa1 = 0.f, ta0 = 0.f, ta1 = 0.f, sb0 = 0.f, sb1 = 0.f, tb0 = 0.f, tb1 = 0.f;
  const float4 *xl = xq, *xh = xq + 8 * stride4;
#pragma unroll 1
  for (int it = 0; it < 4; ++it) {
    const float4 l0 = xl[0], h0 = xh[0], l1 = xl[stride4], h1 = xh[stride4];
    word_fma(a0, l0, h0, sa0, sa1);
    word_fma(b0, l0, h0, sb0, sb1);
    word_fma(a1, l1, h1, ta0, ta1);
    word_fma(b1, l1, h1, tb0, tb1);
    a0 = a2; a1 = a3; a2 = a4; a3 = a5; a4 = a6; a5 = a7;
    b0 = b2; b1 = b3; b2 = b4; b3 = b5; b4 = b6; b5 = b7;
    xl += 2 * stride4;
    xh += 2 * stride4;
  }
  A0 = sa0 + ta0;
  A1 = sa1 + ta1;
  B0 = sb0 + tb0;
  B1 = sb1 + tb1;
}

// four rows (two gate/up pairs) over one pass of the vector: the shared-memory reads of the vector are the
// larger part of a row pair's traffic, so sharing them between pairs pays
__device__ __forceinline__ void quarter_dot4(const Quarter &wa, const Quarter &wb, const Quarter &wc, const Quarter &wd,
                                             const float4 *xq, int stride4, float (&S)[8]) {
  unsigned a0 = wa.q0.x, a1 = wa.q0.y, a2 = wa.q0.z, a3 = wa.q0.w, a4 = wa.q1.x, a5 = wa.q1.y, a6 = wa.q1.z, a7 = wa.q1.w;
  unsigned b0 = wb.q0.x, b1 = wb.q0.y, b2 = wb.q0.z, b3 = wb.q0.w, b4 = wb.q1.x, b5 = wb.q1.y, b6 = wb.q1.z, b7 = wb.q1.w;
  unsigned c0 = wc.q0.x, c1 = wc.q0.y, c2 = wc.q0.z, c3 = wc.q0.w, c4 = wc.q1.x, c5 = wc.q1.y, c6 = wc.q1.z, c7 = wc.q1.w;
  unsigned d0 = wd.q0.x, d1 = wd.q0.y, d2 = wd.q0.z, d3 = wd.q0.w, d4 = wd.q1.x, d5 = wd.q1.y, d6 = wd.q1.z, d7 = wd.q1.w;
#pragma unroll
  for (int i = 0; i < 8; ++i) S[i] = 0.f;
  const float4 *xl = xq, *xh = xq + 8 * stride4;
#pragma unroll 1
  for (int it = 0; it < 4; ++it) {
    const float4 l0 = xl[0], h0 = xh[0], l1 = xl[stride4], h1 = xh[stride4];
    word_fma(a0, l0, h0, S[0], S[1]);
    word_fma(b0, l0, h0, S[2], S[3]);
    word_fma(c0, l0, h0, S[4], S[5]);
    word_fma(d0, l0, h0, S[6], S[7]);
    word_fma(a1, l1, h1, S[0], S[1]);
    word_fma(b1, l1, h1, S[2], S[3]);
    word_fma(c1, l1, h1, S[4], S[5]);
    word_fma(d1, l1, h1, S[6], S[7]);
    a0 = a2; a1 = a3; a2 = a4; a3 = a5; a4 = a6; a5 = a7;
    b0 = b2; b1 = b3; b2 = b4; b3 = b5; b4 = b6; b5 = b7;
    c0 = c2; c1 = c3; c2 = c4; c3 = c5; c4 = c6; c5 = c7;
    d0 = d2; d1 = d3; d2 = d4; d3 = d5; d4 = d6; d5 = d7;
    xl += 2 * stride4;
    xh += 2 * stride4;
  }
}

// position of element k of a vector with Q quarters in its transposed shared-memory form:
// float4 number (i*Q + q) holds elements 64q + 4i .. 64q + 4i + 3
__device__ __forceinline__ int tpos(int k, int Q) {
  const int q = k >> 6, r = k & 63;
  return (((r >> 2) * Q + q) << 2) + (r & 3);
}

__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Shared-memory plan (byte offsets). `slots` gate/up row pairs are staged per warp at a time.
struct Plan {
  uint32_t xs, xsum, wr, nw, small, ypart, asum, av, wstage, total;
};
__host__ __device__ inline Plan make_plan(int T, int H, int F, int k, int slots) {
  const uint32_t P = (uint32_t)(T * k);
  Plan pl;
  uint32_t o = 0;
  auto take = [&](uint32_t bytes) { const uint32_t at = o; o += (bytes + 15u) & ~15u; return at; };
  pl.xs = take((uint32_t)T * H * 4);
  pl.xsum = take((uint32_t)T * (H / 32) * 4);
  pl.wr = take((uint32_t)H * 2);
  pl.nw = take((uint32_t)H * 2);
  pl.small = take(1024);
  pl.ypart = take((uint32_t)kWarps * P * (F / 64 + 1) * 4);
  pl.asum = take(P * (F / 32) * 4);
  pl.av = take(P * F * 4);
  pl.wstage = take((uint32_t)kWarps * slots * 2 * (H / 256) * KNJ_Q4K_BYTES);
  pl.total = o;
  return pl;
}

__global__ void __launch_bounds__(kThreads, 1) moe_stack_small_kernel(const StackParams p) {
  extern __shared__ __align__(16) uint8_t smem_b[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int T = p.T, H = p.H, F = p.F, E = p.E, k = p.k, P = T * k;
  const int QH = H / 64, QF = F / 64;  // quarters per row of gate/up and of down
  const int nslice = H / 256;
  const int G = gridDim.x, c = blockIdx.x;
  const Plan pl = make_plan(T, H, F, k, p.slots);
  float *xs = reinterpret_cast<float *>(smem_b + pl.xs), *xsum = reinterpret_cast<float *>(smem_b + pl.xsum);
  const uint8_t *wr_s = smem_b + pl.wr, *nw_s = smem_b + pl.nw;
  int *sel_e = reinterpret_cast<int *>(smem_b + pl.small);
  int *pair_d = sel_e + 32, *list = sel_e + 64, *ord = sel_e + 96;
  unsigned *dmask = reinterpret_cast<unsigned *>(sel_e + 128), *bitmap = dmask + 32;
  float *sel_w = reinterpret_cast<float *>(sel_e + 176), *scale_s = sel_w + 32;
  int *n_distinct = sel_e + 220;
  float *ypart = reinterpret_cast<float *>(smem_b + pl.ypart), *asum = reinterpret_cast<float *>(smem_b + pl.asum);
  float *av = reinterpret_cast<float *>(smem_b + pl.av);
  uint8_t *wstage = smem_b + pl.wstage;
  unsigned arrivals = 0;
  const unsigned mF = div_magic(F), mQF = div_magic(QF), mF4 = div_magic(F / 4), mH4 = div_magic(H / 4);

  // this CTA's router row and the norm weights of a layer, copied to shared memory ahead of their use
  auto prefetch_router = [&](const StackLayer &Ln) {
    const int chunks = H / 8;  // 16-byte pieces of a bf16 row
    for (int i = threadIdx.x; i < 2 * chunks; i += kThreads) {
      if (i < chunks) {
        if (c < E) cp_async16(smem_b + pl.wr + 16 * i, reinterpret_cast<const uint8_t *>(Ln.Wr) + ((size_t)c * H) * 2 + 16 * i);
      } else if (Ln.norm_w) {
        cp_async16(smem_b + pl.nw + 16 * (i - chunks), reinterpret_cast<const uint8_t *>(Ln.norm_w) + 16 * (i - chunks));
      }
    }
    cp_async_commit();
  };
  prefetch_router(p.layers[0]);

  // the layers' descriptions: read from shared memory where needed instead of held in registers; the next
  // layer's arrives while the current one computes
  __shared__ StackLayer s_layer[2];
  static_assert(sizeof(StackLayer) % 4 == 0, "copied by words");
  auto stage_layer = [&](int l) {
    if (threadIdx.x < sizeof(StackLayer) / 4)
      reinterpret_cast<uint32_t *>(&s_layer[l & 1])[threadIdx.x] = reinterpret_cast<const uint32_t *>(p.layers + l)[threadIdx.x];
  };
  stage_layer(0);
  __syncthreads();
  for (int l = 0; l < p.n_layers; ++l) {
    const StackLayer &L = s_layer[l & 1];
    const bool xf32 = L.x_dtype == KNJ_DT_F32;
    const bool has_norm = L.norm_w != nullptr;

    // ---- loads first, conversions later: the rows come from L2 (another SM wrote them) and a use right after
    // the load would serialise the round trips
    uint4 xr[8];  // warps < T: a bf16 row is fetched whole before it is used; f32 rows (first layer at most) load in place
    if (warp < T && !xf32) {
#pragma unroll
      for (int sl = 0; sl < 8; ++sl)
        if (sl < nslice) xr[sl] = ldcg16(static_cast<const unsigned short *>(L.x) + (int64_t)warp * L.ldx + 256 * sl + 8 * lane);
    }
    // every thread's share of the rows for the transposed copy (4 elements per group), still as loaded
    const int groups = T * (H / 4);
    uint4 xraw[kMaxT];
#pragma unroll
    for (int r = 0; r < kMaxT; ++r) {
      const int g = threadIdx.x + kThreads * r;
      xraw[r] = make_uint4(0u, 0u, 0u, 0u);
      if (g < groups) {
        const int t = fast_div(g, mH4), k4 = g - t * (H / 4);
        const int64_t at = (int64_t)t * L.ldx + 4 * k4;
        if (xf32) {
          xraw[r] = ldcg16(static_cast<const float *>(L.x) + at);
        } else {
          const uint2 r0 = __ldcg(reinterpret_cast<const uint2 *>(static_cast<const unsigned short *>(L.x) + at));
          xraw[r].x = r0.x;
          xraw[r].y = r0.y;
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();  // the router row and the norm weights are in shared memory

    // ---- row statistics of every token (each CTA for itself) and, in CTA e < E, expert e's logits.
    // Operation order of moe_front_kernel: lane owns elements 256*sl + 8*lane + j, even/odd chains, warp_sum.
    if (warp < T) {
      const int t = warp;
      const bool mine = c < E;

      float d0 = 0.f, d1 = 0.f, s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int sl = 0; sl < 8; ++sl) {
        if (sl < nslice) {
          float v[8], wr[8];
          if (xf32) {
            const float *xp = static_cast<const float *>(L.x) + (int64_t)t * L.ldx + 256 * sl + 8 * lane;
            const uint4 r0 = ldcg16(xp), r1 = ldcg16(xp + 4);
            v[0] = __uint_as_float(r0.x); v[1] = __uint_as_float(r0.y); v[2] = __uint_as_float(r0.z); v[3] = __uint_as_float(r0.w);
            v[4] = __uint_as_float(r1.x); v[5] = __uint_as_float(r1.y); v[6] = __uint_as_float(r1.z); v[7] = __uint_as_float(r1.w);
          } else {
            const unsigned u[4] = {xr[sl].x, xr[sl].y, xr[sl].z, xr[sl].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[2 * j] = __uint_as_float(u[j] << 16);
              v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
            }
          }
          if (mine) {
            const uint4 r = *reinterpret_cast<const uint4 *>(wr_s + (256 * sl + 8 * lane) * 2);
            const unsigned u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              wr[2 * j] = __uint_as_float(u[j] << 16);
              wr[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
            }
            if (has_norm) {
              const uint4 rn = *reinterpret_cast<const uint4 *>(nw_s + (256 * sl + 8 * lane) * 2);
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
      }
      const float dot = warp_sum(d0 + d1), ss = warp_sum(s0 + s1);
      if (lane == 0) {
        const float scale = has_norm ? 1.0f / sqrtf(ss / (float)H + L.eps) : 1.0f;
        scale_s[t] = scale;
        if (mine) {
          const float bias = L.bias ? L.bias[c] : 0.f;
          p.logits[(size_t)t * E + c] = dot * scale + bias;
        }
      }
    }
    arrivals += G;
    // this CTA's logits are out: the other CTAs need nothing else from it before the top-k
    grid_arrive(p.sync);
    // ---- the rows the experts see, transposed in shared memory, and their 32-element sums
    // (scale_s was written before the barrier's first CTA-wide synchronisation)
#pragma unroll
    for (int r = 0; r < kMaxT; ++r) {
      const int g = threadIdx.x + kThreads * r;
      if (r * kThreads < groups) {  // whole warps take part in the shuffles
        float4 v;
        if (xf32) v = make_float4(__uint_as_float(xraw[r].x), __uint_as_float(xraw[r].y), __uint_as_float(xraw[r].z), __uint_as_float(xraw[r].w));
        else v = make_float4(__uint_as_float(xraw[r].x << 16), __uint_as_float(xraw[r].x & 0xffff0000u), __uint_as_float(xraw[r].y << 16),
                             __uint_as_float(xraw[r].y & 0xffff0000u));
        int t = 0, k4 = 0;
        if (g < groups) {
          t = fast_div(g, mH4);
          k4 = g - t * (H / 4);
          if (has_norm) {
            const float sc = scale_s[t];
            const uint2 nw = *reinterpret_cast<const uint2 *>(nw_s + 8 * k4);
            v.x = __fmul_rn(__fmul_rn(v.x, sc), __uint_as_float(nw.x << 16));
            v.y = __fmul_rn(__fmul_rn(v.y, sc), __uint_as_float(nw.x & 0xffff0000u));
            v.z = __fmul_rn(__fmul_rn(v.z, sc), __uint_as_float(nw.y << 16));
            v.w = __fmul_rn(__fmul_rn(v.w, sc), __uint_as_float(nw.y & 0xffff0000u));
          }
          *reinterpret_cast<float4 *>(xs + (size_t)t * H + tpos(4 * k4, QH)) = stage_scale(v, (k4 & 8) != 0);
        }
        float s = (v.x + v.y) + (v.z + v.w);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (g < groups && (lane & 7) == 0) xsum[t * (H / 32) + (k4 >> 3)] = s;
      }
    }
    if (!grid_wait(p.sync, arrivals + (l == 0 ? (unsigned)p.stall : 0u), p.spin_limit)) return;

    // ---- top-k per token (every CTA for itself), then the distinct experts in ascending order
    if (warp < T) {
      int se[8];
      float sw[8];
      if (E <= 128) warp_topk<4>(p.logits + (size_t)warp * E, E, k, lane, se, sw);
      else warp_topk(p.logits + (size_t)warp * E, E, k, lane, se, sw);
      if (lane == 0) {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s >= k) break;
          sel_e[warp * k + s] = se[s];
          sel_w[warp * k + s] = sw[s];
          if (c == 0 && L.tap_exp) L.tap_exp[warp * k + s] = se[s];
          if (c == 0 && L.tap_w) L.tap_w[warp * k + s] = sw[s];
        }
      }
    }
    if (warp == kWarps - 1 && lane < 8) bitmap[lane] = 0u;
    __syncthreads();
    if (warp == 0) {
      const int e = lane < P ? sel_e[lane] : -1 - lane;  // distinct dummies so that they match nobody
      if (lane < P) atomicOr(&bitmap[e >> 5], 1u << (e & 31));
      __syncwarp();
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      const bool first = lane < P && (peers & ((1u << lane) - 1u)) == 0u;
      if (lane < P) {
        int d = 0, tot = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          const unsigned m = bitmap[w];
          tot += __popc(m);
          if (w < (e >> 5)) d += __popc(m);
          else if (w == (e >> 5)) d += __popc(m & ((1u << (e & 31)) - 1u));
        }
        pair_d[lane] = d;
        if (first) {
          list[d] = e;
          dmask[d] = peers;
        }
        if (lane == 0) *n_distinct = tot;
        // a token's slots in ascending expert order (the order of the weighted sum)
        const int t = lane / k;
        int r = 0;
        for (int j = 0; j < k; ++j) r += sel_e[t * k + j] < e ? 1 : 0;
        ord[t * k + r] = lane;
      }
    }
    __syncthreads();
    const int D = *n_distinct;

    // ---- gate/up + SiLU*up: row pairs [u0, u1) of this CTA; a warp stages up to `slots` pairs at a time
    {
      const long long U = (long long)D * F;
      const int u0 = (int)(U * c / G), u1 = (int)(U * (c + 1) / G);
      const bool live = lane < QH;
      const int row_bytes = nslice * KNJ_Q4K_BYTES, pair_bytes = 2 * row_bytes, chunks = row_bytes / 16;
      const int S = p.slots;
      uint8_t *wbuf = wstage + (size_t)warp * S * pair_bytes;
      for (int ub = u0 + warp; ub < u1; ub += kWarps * S) {
#pragma unroll
        for (int s = 0; s < 3; ++s) {
          const int u = ub + s * kWarps;
          if (s < S && u < u1) {
            const int d = fast_div(u, mF), n = u - d * F;
            const size_t row = ((size_t)list[d] * F + n) * row_bytes;
            uint8_t *dst = wbuf + s * pair_bytes;
            for (int ch = lane; ch < chunks; ch += 32) {
              cp_async16(dst + 16 * ch, L.Wg + row + 16 * ch);
              cp_async16(dst + row_bytes + 16 * ch, L.Wu + row + 16 * ch);
            }
          }
          cp_async_commit();
        }
        for (int s = 0; s < 3; ++s) {
          const int u = ub + s * kWarps;
          if (s == 0) cp_async_wait<2>();
          else if (s == 1) cp_async_wait<1>();
          else cp_async_wait<0>();
          __syncwarp();
          if (T == 1 && s == 0 && S > 1 && u + kWarps < u1) {
            // one token: slots 0 and 1 go over the vector together
            cp_async_wait<1>();
            __syncwarp();
            const int e0 = fast_div(u, mF), e1 = fast_div(u + kWarps, mF);
            const int n0 = u - e0 * F, n1 = u + kWarps - e1 * F;
            const int pr0 = __ffs(dmask[e0]) - 1, pr1 = __ffs(dmask[e1]) - 1;  // the token's slot that chose the expert
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (live) {
              const uint8_t *sb = wbuf + (lane >> 2) * KNJ_Q4K_BYTES;
              const int qo = KNJ_Q4K_OFF_QS + 32 * (lane & 3);
              Quarter w[4];
#pragma unroll
              for (int r = 0; r < 4; ++r) {
                const uint8_t *rp = sb + r * row_bytes;  // gate 0, up 0, gate 1, up 1
                w[r].hdr = *reinterpret_cast<const uint4 *>(rp);
                w[r].q0 = *reinterpret_cast<const uint4 *>(rp + qo);
                w[r].q1 = *reinterpret_cast<const uint4 *>(rp + qo + 16);
              }
              float S8[8];
              quarter_dot4(w[0], w[1], w[2], w[3], reinterpret_cast<const float4 *>(xs) + lane, QH, S8);
              const float x0 = xsum[2 * lane], x1 = xsum[2 * lane + 1];
#pragma unroll
              for (int r = 0; r < 4; ++r) {
                float a0, b0, a1, b1;
                quarter_scales(w[r].hdr, lane & 3, a0, b0, a1, b1);
                v[r] = (a0 * S8[2 * r] + a1 * S8[2 * r + 1]) - (b0 * x0 + b1 * x1);
              }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
              for (int r = 0; r < 4; ++r) v[r] += __shfl_xor_sync(0xffffffffu, v[r], o);
            }
            if (lane == 0) {
              p.act[(size_t)pr0 * F + n0] = (v[0] / (1.0f + expf(-v[0]))) * v[1];
              p.act[(size_t)pr1 * F + n1] = (v[2] / (1.0f + expf(-v[2]))) * v[3];
            }
            s = 1;  // slot 1 is done too
            continue;
          }
          if (s < S && u < u1) {
            const int d = fast_div(u, mF), n = u - d * F;
            const uint8_t *slot = wbuf + s * pair_bytes;
            Quarter wg, wu;
            float ga0 = 0.f, gb0 = 0.f, ga1 = 0.f, gb1 = 0.f, ua0 = 0.f, ub0 = 0.f, ua1 = 0.f, ub1 = 0.f;
            if (live) {
              const uint8_t *sb = slot + (lane >> 2) * KNJ_Q4K_BYTES;
              wg.hdr = *reinterpret_cast<const uint4 *>(sb);
              wg.q0 = *reinterpret_cast<const uint4 *>(sb + KNJ_Q4K_OFF_QS + 32 * (lane & 3));
              wg.q1 = *reinterpret_cast<const uint4 *>(sb + KNJ_Q4K_OFF_QS + 32 * (lane & 3) + 16);
              wu.hdr = *reinterpret_cast<const uint4 *>(sb + row_bytes);
              wu.q0 = *reinterpret_cast<const uint4 *>(sb + row_bytes + KNJ_Q4K_OFF_QS + 32 * (lane & 3));
              wu.q1 = *reinterpret_cast<const uint4 *>(sb + row_bytes + KNJ_Q4K_OFF_QS + 32 * (lane & 3) + 16);
              quarter_scales(wg.hdr, lane & 3, ga0, gb0, ga1, gb1);
              quarter_scales(wu.hdr, lane & 3, ua0, ub0, ua1, ub1);
            }
            unsigned todo = dmask[d];
            while (todo) {
              const int pr = __ffs(todo) - 1;
              todo &= todo - 1u;
              const int t = (pr >= k) + (pr >= 2 * k) + (pr >= 3 * k);  // pr / k for at most four tokens
              float vg = 0.f, vu = 0.f;
              if (live) {
                float A0, A1, B0, B1;
                quarter_dot2(wg, wu, reinterpret_cast<const float4 *>(xs + (size_t)t * H) + lane, QH, A0, A1, B0, B1);
                const float x0 = xsum[t * (H / 32) + 2 * lane], x1 = xsum[t * (H / 32) + 2 * lane + 1];
                vg = (ga0 * A0 + ga1 * A1) - (gb0 * x0 + gb1 * x1);
                vu = (ua0 * B0 + ua1 * B1) - (ub0 * x0 + ub1 * x1);
              }
              vg = warp_sum(vg);
              vu = warp_sum(vu);
              if (lane == 0) p.act[(size_t)pr * F + n] = (vg / (1.0f + expf(-vg))) * vu;
            }
          }
        }
        __syncwarp();  // the slots are free again
      }
    }
    arrivals += G;
    grid_arrive(p.sync);

    // ---- the down rows this warp will need are known already: fetch them before waiting for the activations
    const int n_lo = (int)((long long)H * c / G), n_hi = (int)((long long)H * (c + 1) / G);
    const int tasks = D * QF;  // (distinct expert, quarter) pairs of one output column
    const size_t drow_bytes = (size_t)(F / 256) * KNJ_Q4K_BYTES;
    const int my_col = n_lo + warp;
    const bool ahead = my_col < n_hi;
    Quarter dq0, dq1, dq2;  // tasks lane, lane + 32, lane + 64 of the warp's first column
    auto down_row = [&](int j, int n) {
      const int d = fast_div(j, mQF);
      return L.Wd + ((size_t)list[d] * H + n) * drow_bytes;
    };
    if (ahead) {
      if (lane < tasks) load_quarter(down_row(lane, my_col), lane - fast_div(lane, mQF) * QF, dq0);
      if (lane + 32 < tasks) load_quarter(down_row(lane + 32, my_col), lane + 32 - fast_div(lane + 32, mQF) * QF, dq1);
      if (lane + 64 < tasks) load_quarter(down_row(lane + 64, my_col), lane + 64 - fast_div(lane + 64, mQF) * QF, dq2);
    }

    if (!grid_wait(p.sync, arrivals, p.spin_limit)) return;
    if (l + 1 < p.n_layers) {
      prefetch_router(p.layers[l + 1]);
      stage_layer(l + 1);  // published by the CTA-wide synchronisations below
    }

    // ---- activations of all pairs, transposed, and their 32-element sums
    {
      const int agroups = P * (F / 4);
      constexpr int kAhead = 3;  // loads in flight per thread
      for (int g0 = 0; g0 < agroups; g0 += kThreads * kAhead) {
        uint4 r0[kAhead];
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
          const int g = g0 + a * kThreads + threadIdx.x;
          r0[a] = make_uint4(0u, 0u, 0u, 0u);
          if (g < agroups) r0[a] = ldcg16(p.act + (size_t)4 * g);  // pair rows are contiguous: group g is floats 4g..4g+3
        }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
          const int g = g0 + a * kThreads + threadIdx.x;
          if (g0 + a * kThreads < agroups) {  // whole warps take part in the shuffles
            const float4 v = make_float4(__uint_as_float(r0[a].x), __uint_as_float(r0[a].y), __uint_as_float(r0[a].z), __uint_as_float(r0[a].w));
            int pr = 0, k4 = 0;
            if (g < agroups) {
              pr = fast_div(g, mF4);
              k4 = g - pr * (F / 4);
              *reinterpret_cast<float4 *>(av + (size_t)pr * F + tpos(4 * k4, QF)) = stage_scale(v, (k4 & 8) != 0);
            }
            float s = (v.x + v.y) + (v.z + v.w);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (g < agroups && (lane & 7) == 0) asum[pr * (F / 32) + (k4 >> 3)] = s;
          }
        }
      }
    }
    __syncthreads();

    // ---- down + ordered combine + residual: one output column per warp
    float *yp = ypart + (size_t)warp * P * (QF + 1);
    for (int n = my_col; n < n_hi; n += kWarps) {
      // the residual element comes from L2: asked for now, used after the products
      float resid = 0.f;
      if (L.residual && lane < T) resid = ldcg_as_f32(L.x, L.x_dtype, (int64_t)lane * L.ldx + n);
      for (int r = 0; r * 32 < tasks; ++r) {
        const int j = lane + 32 * r;
        if (j < tasks) {
          const int d = fast_div(j, mQF), q = j - d * QF;
          Quarter w;
          if (n == my_col && r < 3) w = r == 0 ? dq0 : (r == 1 ? dq1 : dq2);
          else load_quarter(down_row(j, n), q, w);
          float a0, b0, a1, b1;
          quarter_scales(w.hdr, q & 3, a0, b0, a1, b1);
          unsigned todo = dmask[d];
          while (todo) {
            const int pr = __ffs(todo) - 1;
            todo &= todo - 1u;
            float S0, S1;
            quarter_dot(w, reinterpret_cast<const float4 *>(av + (size_t)pr * F) + q, QF, S0, S1);
            const float x0 = asum[pr * (F / 32) + 2 * q], x1 = asum[pr * (F / 32) + 2 * q + 1];
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
          const int pr = ord[lane * k + s];
          acc = __fadd_rn(acc, __fmul_rn(sel_w[pr], yp[pr * (QF + 1) + QF]));
        }
        if (L.residual) acc = __fadd_rn(resid, acc);
        store_from_f32(L.out, L.out_dtype, (int64_t)lane * L.ldo + n, acc);
      }
      __syncwarp();
    }

    arrivals += G;
    if (l + 1 < p.n_layers && !grid_barrier(p.sync, arrivals, p.spin_limit)) return;
  }
  cp_async_wait<0>();
}

}  // namespace

namespace knj {
struct SmallStack {
  StackParams p{};
  void *dev_block = nullptr;  // layer table, logits, activations, sync words
  size_t smem = 0;
  int grid = 0;
  int device = 0;
};

int small_stack_create(const knj_moe_ffn_args *layers, int n_layers, SmallStack **out) {
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
  int device = 0;
  KNJ_CUDA(cudaGetDevice(&device));
  SmallStack *st = new SmallStack();
  st->device = device;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, st->device) != cudaSuccess) {
    cudaGetLastError();
    delete st;
    set_error("knj_moe_stack_create: the device's properties cannot be read");
    return KNJ_E_RUNTIME;
  }
  st->p.slots = 1;
  for (int sl = 3; sl >= 1; --sl)
    if (make_plan(T, H, F, k, sl).total <= (size_t)prop.sharedMemPerBlockOptin) { st->p.slots = sl; break; }
  st->smem = make_plan(T, H, F, k, st->p.slots).total;
  if (!prop.cooperativeLaunch || st->smem > (size_t)prop.sharedMemPerBlockOptin) {
    set_error("knj_moe_stack_create: the device lacks cooperative launch or %zu bytes of shared memory per block", st->smem);
    delete st;
    return KNJ_E_REFUSE;
  }
  cudaError_t e = cudaFuncSetAttribute(moe_stack_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st->smem);
  int per_sm = 0;
  if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_stack_small_kernel, kThreads, st->smem);
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
  st->p.spin_limit = kMaxWaitCycles;
  st->p.stall = 0;
  *out = st;
  return KNJ_OK;
}

int small_stack_launch(SmallStack *st, knj_stream_t s) {
  KNJ_REQUIRE(st && st->dev_block, "knj_moe_stack_decode_launch: null stack");
  KNJ_CUDA(cudaMemsetAsync(st->p.sync, 0, 8, as_stream(s)));
  void *args[] = {&st->p};
  KNJ_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(moe_stack_small_kernel), dim3(st->grid), dim3(kThreads), args,
                                       st->smem, as_stream(s)));
  return launch_status("moe_stack_small_kernel");
}

void small_stack_set_wait(SmallStack *st, long long cycles, int stall) {
  st->p.spin_limit = cycles;
  st->p.stall = stall;
}

int small_stack_status(SmallStack *st, knj_stream_t s) {
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

void small_stack_destroy(SmallStack *st) {
  if (!st) return;
  if (st->dev_block) cudaFree(st->dev_block);
  delete st;
}

}  // namespace knj
