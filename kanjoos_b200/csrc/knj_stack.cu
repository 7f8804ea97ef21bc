// knj_stack.cu -- the resident decode stack (RMSNorm -> router -> top-k -> gate/up
// -> SiLU*up -> down -> ordered combine -> residual, layer after layer) for a decode
// batch of 1..64 tokens in ONE cooperative launch. The reference runs this loop on
// the host, one stage at a time (src/model/model.cpp:399-510 per layer, the device
// benches tools/bench/q4k_stream_ffn.hip:957-1313 between kernels).
//
// Why: a decode layer reads 21 MB (batch 1) to 340 MB (batch 64), 3 to 53 us of HBM
// time, but a chain of separate kernels pays a launch, a plan read and several
// dependent round trips per stage. Here the whole stack is one grid of one CTA per
// SM, and the four points per layer at which every CTA needs what the others
// produced (logits -> top-k, activations -> down, per-pair rows -> combine, layer
// output -> next layer) are grid barriers on a counter in global memory.
//
// Arithmetic. Logits and RMS statistics repeat moe_front_kernel's operation order
// exactly, so routing decisions are the same bits as the layer launches'. The expert
// projections run on the tile engine of knj_q4k_engine.cuh (exact integer products
// on the fp16 tensor cores, f32 results); the combine adds the k weighted rows of a
// token in ascending expert order from zero and the residual last, like
// combine_kernel and the CPU path (src/model/model.cpp:455-463, :652).
//
// Every wait is bounded: a barrier or a copy that does not complete within the
// limit sets the error word, every CTA that sees it returns, and
// knj_moe_stack_status reports KNJ_E_TIMEOUT.
#include "knj_common.cuh"
#include "knj_q4k.h"
#include "knj_q4k_engine.cuh"
#include "knj_q6k_block.cuh"
#include "knj_topk.cuh"

#include <algorithm>
#include <vector>

using namespace knj;

namespace {

constexpr int kMaxT = 64;  // tokens per step
constexpr int kThreads = q4e::kWarps * 32;
constexpr int kSplitMaxT = 16;  // batches up to this size may split a tile's K range over several warps
constexpr int kMaxSlices = 8;  // hidden <= 2048: the logits keep a router row in registers

struct LayerMaps {  // stay in global memory: the TMA unit reads them there
  CUtensorMap mg, mu, md;  // gate, up, down weights as TMA boxes of the projection phases
};
struct LayerDesc {  // copied to shared memory one layer ahead
  const void *x;
  void *out;
  const __nv_bfloat16 *Wr;
  const float *bias;
  const __nv_bfloat16 *norm_w;
  const uint8_t *w_down6;  // non-null: the layer's down matrices are Q6_K [E][H][F/256][210] (no TMA map for them)
  int32_t *tap_exp;
  float *tap_w;
  int64_t ldx, ldo;
  float eps;
  int residual, x_dtype, out_dtype;
};
static_assert(sizeof(LayerDesc) % 4 == 0, "copied by words");

struct StackParams {
  const LayerMaps *maps;
  const LayerDesc *layers;
  int n_layers, T, H, F, E, k;
  float *logits;       // [T][E]
  float *scales;       // [T] RMSNorm scale of the layer's rows
  float *act;          // [T*k][F]
  float *Y;            // [T*k][H]
  unsigned int *sync;  // [0] arrivals, [1] error word; both zero before the launch
  q4e::PhaseShape gu, dn;
  long long wait_cycles;  // limit of every wait inside the kernel
  int stall;              // test hook: added to the first barrier's target, which then cannot complete
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

// Shared-memory plan (byte offsets into the dynamic block).
struct Plan {
  uint32_t ring, panels, bars, sel_e, sel_w, mask, jbase, uexp, inv, pair, scale, ord, fail, desc, red, total;
};
__host__ __device__ inline Plan make_plan(const q4e::PhaseShape &gu, const q4e::PhaseShape &dn, int T, int k) {
  Plan pl;
  uint32_t o = 0;
  auto take = [&](size_t bytes) { const uint32_t at = o; o += (uint32_t)((bytes + 127) & ~(size_t)127); return at; };
  const size_t ring = max(q4e::phase_ring_bytes(gu.sbs, gu.stages), q4e::phase_ring_bytes(dn.sbs, dn.stages));
  const size_t panels = max(q4e::phase_panel_bytes(gu.nsb), q4e::phase_panel_bytes(dn.nsb));
  pl.ring = take(ring);
  pl.panels = take(panels);
  pl.bars = take((size_t)q4e::kWarps * q4e::kMaxStages * 8);
  pl.sel_e = take((size_t)T * k * 4);
  pl.sel_w = take((size_t)T * k * 4);
  pl.mask = take(256 * 8);
  pl.jbase = take(257 * 4);
  pl.uexp = take(256 * 4);
  pl.inv = take(q4e::kJobTok * 16 * 4);
  pl.pair = take(q4e::kJobTok * 4);
  pl.scale = take((size_t)T * 4);
  pl.ord = take((size_t)T * k);
  pl.fail = take(32);   // fail word, then the two block barriers of the Q6_K down phase
  pl.desc = take(2 * sizeof(LayerDesc));
  // partial sums of warps that share a tile: only small batches have so few tiles that they do
  pl.red = T <= kSplitMaxT ? take((size_t)q4e::kWarps * 32 * sizeof(float4)) : 0;
  pl.total = o;
  return pl;
}

__device__ __forceinline__ void load8_bf16(const __nv_bfloat16 *p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4 *>(p));
  const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(u[j] << 16);
    v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
  }
}

#ifdef KNJ_TRACE
// Measurement build only: global-timer stamps of one CTA's stages in layer 1 (layer 0 of a one-layer stack).
__device__ unsigned long long g_stack_trace[16 * 160];
#define KNJ_STAMP(i) do { if (threadIdx.x == 0 && l == trace_layer) g_stack_trace[blockIdx.x * 16 + (i)] = global_timer_ns(); } while (0)
#else
#define KNJ_STAMP(i)
#endif

// Stage 1 of a layer for one CTA item: experts epi * eg .. + epi - 1 times tokens 8 tg .. 8 tg + 7; warp w takes
// expert w % epi and the token slot w / epi (epi / 2 tokens, at least one). epi = 8, 4, 2 or 1: fewer experts per
// item for smaller batches, so that the items still cover most of the grid. Row statistics and logits in moe_front_kernel's operation order (lane owns
// elements 256 sl + 8 lane + j, even/odd chains, warp_sum). The CTA first brings its eight router rows (times the
// norm weights, f32) and its token rows (as they are) into shared memory with every load in flight at once;
// scratch: 8 * H * 4 bytes for the router rows followed by 8 * H * 4 for the token rows.
__device__ __noinline__ void stage_logits(const StackParams &p, const LayerDesc &L, int epi, int eg, int tg, uint8_t *scratch,
                                          int l, int trace_layer) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int T = p.T, H = p.H, E = p.E, nslice = H / 256;
  const bool has_norm = L.norm_w != nullptr;
  float *wr_s = reinterpret_cast<float *>(scratch);
  uint8_t *rows_s = scratch + (size_t)8 * H * 4;
  const int esz = L.x_dtype == KNJ_DT_F32 ? 4 : 2, row_bytes = H * esz, cpr = row_bytes / 16;
  const int nt = min(8, T - tg * 8);
  // ---- loads first (router rows, norm weights, token rows), conversions after
  const int wchunks = epi * (H / 8);  // 16-byte pieces of the item's bf16 router rows
  constexpr int kPer = (8 * 256 * kMaxSlices / 8 + kThreads - 1) / kThreads;  // 4 pieces per thread at H = 2048
  uint4 wraw[kPer], nraw[kPer];
#pragma unroll
  for (int q = 0; q < kPer; ++q) {
    const int i = threadIdx.x + q * kThreads;
    if (i < wchunks) {
      const int r = i / (H / 8), ch = i - r * (H / 8);
      const int ee = min(eg * epi + r, E - 1);
      wraw[q] = __ldg(reinterpret_cast<const uint4 *>(L.Wr + (size_t)ee * H + 8 * ch));
      if (has_norm) nraw[q] = __ldg(reinterpret_cast<const uint4 *>(L.norm_w + 8 * ch));
    }
  }
  for (int i = threadIdx.x; i < nt * cpr; i += kThreads) {
    const int r = i / cpr, ch = i - r * cpr;
    *reinterpret_cast<uint4 *>(rows_s + (size_t)r * row_bytes + 16 * ch) =
        __ldcg(reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(L.x) + (int64_t)(tg * 8 + r) * L.ldx * esz + 16 * ch));
  }
#pragma unroll
  for (int q = 0; q < kPer; ++q) {
    const int i = threadIdx.x + q * kThreads;
    if (i < wchunks) {
      const uint32_t w[4] = {wraw[q].x, wraw[q].y, wraw[q].z, wraw[q].w}, n[4] = {nraw[q].x, nraw[q].y, nraw[q].z, nraw[q].w};
      float v[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        if (has_norm) {
          v[2 * j] *= __uint_as_float(n[j] << 16);
          v[2 * j + 1] *= __uint_as_float(n[j] & 0xffff0000u);
        }
      }
      *reinterpret_cast<float4 *>(wr_s + (size_t)8 * i) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4 *>(wr_s + (size_t)8 * i + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  __syncthreads();
  KNJ_STAMP(11);
  const int es = warp % epi, tpw = max(1, epi / 2);
  const int e = eg * epi + es;
  const int t_first = tg * 8 + (warp / epi) * tpw, t_end = min(min(T, tg * 8 + 8), t_first + tpw);
  const float bias = (L.bias && e < E) ? L.bias[e] : 0.f;
  const float *wrow = wr_s + (size_t)es * H;
  // two tokens per pass over the router row: their chains are independent of each other
  for (int t = t_first; t < t_end; t += 2) {
    const bool second = t + 1 < t_end;
    float d0[2] = {0.f, 0.f}, d1[2] = {0.f, 0.f}, s0[2] = {0.f, 0.f}, s1[2] = {0.f, 0.f};
#pragma unroll
    for (int sl = 0; sl < kMaxSlices; ++sl) {
      if (sl < nslice) {
        const float4 wa = *reinterpret_cast<const float4 *>(wrow + 256 * sl + 8 * lane);
        const float4 wb = *reinterpret_cast<const float4 *>(wrow + 256 * sl + 8 * lane + 4);
        const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint8_t *row = rows_s + (size_t)(t + (second ? u : 0) - tg * 8) * row_bytes;
          float v[8];
          if (esz == 4) {
            const float4 a = *reinterpret_cast<const float4 *>(row + (256 * sl + 8 * lane) * 4);
            const float4 b = *reinterpret_cast<const float4 *>(row + (256 * sl + 8 * lane) * 4 + 16);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
          } else {
            const uint4 r = *reinterpret_cast<const uint4 *>(row + (256 * sl + 8 * lane) * 2);
            const uint32_t x4[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[2 * j] = __uint_as_float(x4[j] << 16);
              v[2 * j + 1] = __uint_as_float(x4[j] & 0xffff0000u);
            }
          }
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            d0[u] = fmaf(w[j], v[j], d0[u]);
            d1[u] = fmaf(w[j + 1], v[j + 1], d1[u]);
            s0[u] = fmaf(v[j], v[j], s0[u]);
            s1[u] = fmaf(v[j + 1], v[j + 1], s1[u]);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && !second) break;
      const float dot = warp_sum(d0[u] + d1[u]), ss = warp_sum(s0[u] + s1[u]);
      if (lane == 0) {
        const float scale = has_norm ? 1.0f / sqrtf(ss / (float)H + L.eps) : 1.0f;
        if (eg == 0 && es == 0) p.scales[t + u] = scale;
        if (e < E) p.logits[(size_t)(t + u) * E + e] = dot * scale + bias;
      }
    }
  }
}

// Stage 2 of a layer, by every CTA for itself: top-k of every token, the per-expert token sets (bit masks), the
// order of a token's slots for the weighted sum, and the job table of the projection stages.
__device__ __noinline__ void stage_plan(const StackParams &p, const LayerDesc &L, const Plan &pl, uint8_t *smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int T = p.T, E = p.E, k = p.k, P = T * k, c = blockIdx.x;
  int *sel_e = reinterpret_cast<int *>(smem + pl.sel_e);
  float *sel_w = reinterpret_cast<float *>(smem + pl.sel_w);
  unsigned long long *mask = reinterpret_cast<unsigned long long *>(smem + pl.mask);
  int *jbase = reinterpret_cast<int *>(smem + pl.jbase), *uexp = reinterpret_cast<int *>(smem + pl.uexp);
  float *scale_s = reinterpret_cast<float *>(smem + pl.scale);
  unsigned char *ord = smem + pl.ord;
    for (int t = threadIdx.x; t < T; t += kThreads) scale_s[t] = __ldcg(p.scales + t);
    for (int a = threadIdx.x; a < 256; a += kThreads) mask[a] = 0ull;
    for (int t = warp; t < T; t += q4e::kWarps) {
      int se[8];
      float sw[8];
      if (E <= 128) warp_topk<4>(p.logits + (size_t)t * E, E, k, lane, se, sw);
      else warp_topk(p.logits + (size_t)t * E, E, k, lane, se, sw);
      if (lane == 0) {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s >= k) break;
          sel_e[t * k + s] = se[s];
          sel_w[t * k + s] = sw[s];
          if (c == 0 && L.tap_exp) L.tap_exp[t * k + s] = se[s];
          if (c == 0 && L.tap_w) L.tap_w[t * k + s] = sw[s];
        }
      }
    }
    __syncthreads();
    for (int pr = threadIdx.x; pr < P; pr += kThreads) {
      const int t = pr / k, e = sel_e[pr];
      atomicOr(&mask[e], 1ull << t);
      int r = 0;  // a token's slots in ascending expert order (the order of the weighted sum)
      for (int j = 0; j < k; ++j) r += sel_e[t * k + j] < e ? 1 : 0;
      ord[t * k + r] = (unsigned char)(pr - t * k);
    }
    __syncthreads();
    if (warp == 0) {
      int cnt[8], nact = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = 8 * lane + i;
        cnt[i] = e < E ? __popcll(mask[e]) : 0;
        nact += cnt[i] > 0 ? 1 : 0;
      }
      int incl = nact;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int total = __shfl_sync(0xffffffffu, incl, 31);
      int pos = incl - nact;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (cnt[i] > 0) {
          uexp[pos] = 8 * lane + i;
          jbase[pos] = (cnt[i] + q4e::kJobTok - 1) / q4e::kJobTok;
          ++pos;
        }
      for (int a = total + lane; a < 256; a += 32) {
        uexp[a] = -1;
        jbase[a] = 0;
      }
      __syncwarp();
      q4e::job_prefix(jbase, lane);
      if (lane == 0) jbase[259] = total;  // active experts (behind the job table, inside its padding)
    }
    __syncthreads();

}

// Down phase of a layer whose down matrices are Q6_K: (active expert, one to four blocks of 64 output rows) units
// dealt round robin over the CTAs; the blocks' superblocks and the activation side of up to eight of the expert's
// tokens live in the (idle) ring area, the arithmetic is knj_q6k_block.cuh's, i.e. the stand-alone projection's.
// Where the blocks can travel as bulk copies (16-byte aligned base, H a multiple of 64) and the ring area holds two
// of them, the next block is under way while this one is worked on: two barriers behind the fail word, `staged`
// counts this CTA's blocks over the whole launch.
__device__ __noinline__ void stage_down_q6k(const StackParams &p, const LayerDesc &L, const Plan &pl, uint8_t *smem, unsigned &staged,
                                            bool &ok) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int H = p.H, F = p.F, k = p.k, c = blockIdx.x, G = gridDim.x;
  const int *sel_e = reinterpret_cast<const int *>(smem + pl.sel_e);
  const unsigned long long *mask = reinterpret_cast<const unsigned long long *>(smem + pl.mask);
  const int *jbase = reinterpret_cast<const int *>(smem + pl.jbase), *uexp = reinterpret_cast<const int *>(smem + pl.uexp);
  int *s_pair = reinterpret_cast<int *>(smem + pl.inv);  // eight ints: the pass's output rows (the phase engine is idle)
  const int row_bytes = F / KNJ_QK_K * KNJ_Q6K_BYTES;
  const bool two = 2 * q6b::block_bytes(F) + q6b::act_scratch_bytes(F, q4e::kWarps) <= (size_t)(pl.panels - pl.ring);
  const bool bulk = (reinterpret_cast<uintptr_t>(L.w_down6) & 15u) == 0 && H % q6b::kRows == 0;
  const q6b::Bufs b = q6b::carve(smem + pl.ring, F, q4e::kWarps, two, reinterpret_cast<uint64_t *>(smem + pl.fail + 16),
                                 reinterpret_cast<int *>(smem + pl.fail));
  const int blocks = (H + q6b::kRows - 1) / q6b::kRows, n_act = jbase[259];
  const int sub = max(1, min(4, n_act * blocks / (2 * G)));  // blocks per unit: the activation side is prepared once per unit
  const int chunks = (blocks + sub - 1) / sub, total = n_act * chunks;
  for (int u = c; u < total; u += G) {
    const int a = u / chunks, ch = u - a * chunks;
    const int e = uexp[a];
    const int n0 = ch * sub * q6b::kRows, n_rows = min(sub * q6b::kRows, H - n0);
    unsigned long long m = mask[e];
    while (m) {
      __syncthreads();  // the previous pass is done with the shared buffers
      // the pass's tokens are the lowest set bits of the mask: thread 8 i + j looks at slot j (+ 8, ...) of the i-th
      const int nt = min(q6b::kTok, __popcll(m));
      if (threadIdx.x < 8 * q6b::kTok) {
        const int i = threadIdx.x >> 3;
        unsigned long long mm = m;
        for (int x = 0; x < i; ++x) mm &= mm - 1;
        if (i < nt) {
          const int tok = __ffsll((long long)mm) - 1;
          for (int j = threadIdx.x & 7; j < k; j += 8)
            if (sel_e[tok * k + j] == e) s_pair[i] = tok * k + j;
        }
      }
      for (int i = 0; i < nt; ++i) m &= m - 1;
      __syncthreads();
      if (!q6b::chunk_pass<q4e::kWarps>(b, L.w_down6 + ((size_t)e * H + n0) * row_bytes, n_rows, F, p.act, p.Y + n0, H, s_pair, nt, staged,
                                        bulk, p.wait_cycles, lane, warp)) {
        ok = false;  // a copy that never completes: bounded wait, the launch reports it
        m = 0;
        u = total;
      }
    }
  }
  __syncthreads();  // the ring area returns to the projection phases
}

__global__ void __launch_bounds__(kThreads, 1) moe_stack_kernel(const StackParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int T = p.T, H = p.H, F = p.F, E = p.E, k = p.k;
  const int G = gridDim.x, c = blockIdx.x;
  const Plan pl = make_plan(p.gu, p.dn, T, k);
  int *sel_e = reinterpret_cast<int *>(smem + pl.sel_e);
  float *sel_w = reinterpret_cast<float *>(smem + pl.sel_w);
  unsigned long long *mask = reinterpret_cast<unsigned long long *>(smem + pl.mask);
  int *jbase = reinterpret_cast<int *>(smem + pl.jbase), *uexp = reinterpret_cast<int *>(smem + pl.uexp);
  float *scale_s = reinterpret_cast<float *>(smem + pl.scale);
  unsigned char *ord = smem + pl.ord;
  int *s_fail = reinterpret_cast<int *>(smem + pl.fail);
  q4e::PhaseSmem sm;
  sm.ring = smem + pl.ring;
  sm.panels = smem + pl.panels;
  sm.bars = reinterpret_cast<uint64_t *>(smem + pl.bars);
  sm.inv = reinterpret_cast<float *>(smem + pl.inv);
  sm.pair = reinterpret_cast<int *>(smem + pl.pair);
  sm.fail = s_fail;
  sm.red = reinterpret_cast<float4 *>(smem + pl.red);
  const q4e::JobTable jt{jbase, uexp};

  if (lane == 0)
    for (int s = 0; s < q4e::kMaxStages; ++s) mbar_init(&sm.bars[warp * q4e::kMaxStages + s], 1);
  if (threadIdx.x == 0) {
    *s_fail = 0;
    // the Q6_K down phase's two block barriers (behind the fail word)
    mbar_init(reinterpret_cast<uint64_t *>(smem + pl.fail + 16), 1);
    mbar_init(reinterpret_cast<uint64_t *>(smem + pl.fail + 24), 1);
  }
  mbar_init_fence();
  __syncthreads();

  unsigned arrivals = 0, parity = 0;
  bool ok = true;
  unsigned q6_staged = 0;  // Q6_K down blocks this CTA has staged so far (stage_down_q6k)
  // logits: CTA c < n_eg * n_tg takes experts epi * eg .. + epi - 1 for tokens 8 tg .. 8 tg + 7
  const int n_tg = (T + 7) / 8;
  int epi = 8;
  while (epi > 1 && n_tg * ((E + epi / 2 - 1) / (epi / 2)) <= G) epi >>= 1;
  const int n_eg = (E + epi - 1) / epi;
  const bool has_item = c < n_eg * n_tg;
  const int eg = c % n_eg, tg = c / n_eg;

#ifdef KNJ_TRACE
  const int trace_layer = p.n_layers > 1 ? 1 : 0;
#endif
  // the layers' descriptions are read from shared memory; the next layer's arrives while the current one computes
  LayerDesc *descs = reinterpret_cast<LayerDesc *>(smem + pl.desc);
  auto stage_desc = [&](int l) {
    if (threadIdx.x < sizeof(LayerDesc) / 4)
      reinterpret_cast<uint32_t *>(&descs[l & 1])[threadIdx.x] = reinterpret_cast<const uint32_t *>(p.layers + l)[threadIdx.x];
  };
  stage_desc(0);
  __syncthreads();
  for (int l = 0; l < p.n_layers; ++l) {
    const LayerDesc &L = descs[l & 1];
    const LayerMaps &M = p.maps[l];
    const bool has_norm = L.norm_w != nullptr;
    if (l + 1 < p.n_layers) stage_desc(l + 1);  // published by the CTA barriers of this layer
    KNJ_STAMP(0);

    // ---- stage 1: row statistics and router logits
#ifdef KNJ_TRACE
    if (has_item) stage_logits(p, L, epi, eg, tg, smem + pl.ring, l, trace_layer);
#else
    if (has_item) stage_logits(p, L, epi, eg, tg, smem + pl.ring, l, 0);
#endif
    KNJ_STAMP(1);
    arrivals += G;
    grid_arrive(p.sync);
    if (!grid_wait(p.sync, arrivals + (l == 0 ? (unsigned)p.stall : 0u), p.wait_cycles)) return;
    KNJ_STAMP(2);

    // ---- stage 2: top-k per token (every CTA for itself), the per-expert token sets, the job table
    stage_plan(p, L, pl, smem);

    // token slot tk of a job: the (4 (job - first job of the expert) + tk)-th token of the expert's set
    auto job_tok = [&](int job, int a, int tk, int &e_out) {
      const int e = uexp[a];
      unsigned long long m = mask[e];
      const int idx = (job - jbase[a]) * q4e::kJobTok + tk;
      e_out = e;
      if (idx >= __popcll(m)) return -1;
      for (int i = 0; i < idx; ++i) m &= m - 1ull;
      return __ffsll((long long)m) - 1;
    };
    auto pair_of = [&](int tok, int e) {
      int s = 0;
      for (int j = 0; j < k; ++j) s = sel_e[tok * k + j] == e ? j : s;
      return tok * k + s;
    };

    KNJ_STAMP(3);
    // ---- stage 3: gate, up, SiLU*up -> act
    {
      const long long U = (long long)jbase[256] * p.gu.tiles;
      const int u0 = (int)(U * c / G), u1 = (int)(U * (c + 1) / G);
      q4e::run_phase<true>(
          p.gu, sm, jt, u0, u1, T <= kSplitMaxT ? q4e::choose_ksplit(U, p.gu.nsb / p.gu.sbs, G) : 1, &M.mg, &M.mu, nullptr, nullptr, p.act, p.wait_cycles, parity, ok,
          [&](int job, int a, int tk, int &pair, int &row) {
            int e;
            const int tok = job_tok(job, a, tk, e);
            if (tok < 0) return false;
            pair = pair_of(tok, e);
            row = tok;
            return true;
          },
          [&](int row, int sb, int ln, float (&v)[8]) {
            q4e::load8_f32(L.x, L.x_dtype, (int64_t)row * L.ldx + 256 * sb + 8 * ln, v);
            if (has_norm) {
              float nw[8];
              load8_bf16(L.norm_w + 256 * sb + 8 * ln, nw);
              const float sc = scale_s[row];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], sc), nw[j]);
            }
          });
    }
    KNJ_STAMP(4);
    arrivals += G;
    grid_arrive(p.sync);
    if (!grid_wait(p.sync, arrivals, p.wait_cycles)) return;
    KNJ_STAMP(5);

    // ---- stage 4: down -> Y (one row per pair)
    if (L.w_down6) stage_down_q6k(p, L, pl, smem, q6_staged, ok);
    else {
      const long long U = (long long)jbase[256] * p.dn.tiles;
      const int u0 = (int)(U * c / G), u1 = (int)(U * (c + 1) / G);
      q4e::run_phase<false>(
          p.dn, sm, jt, u0, u1, T <= kSplitMaxT ? q4e::choose_ksplit(U, p.dn.nsb / p.dn.sbs, G) : 1, &M.md, &M.md, p.Y, nullptr, nullptr, p.wait_cycles, parity, ok,
          [&](int job, int a, int tk, int &pair, int &row) {
            int e;
            const int tok = job_tok(job, a, tk, e);
            if (tok < 0) return false;
            pair = pair_of(tok, e);
            row = pair;
            return true;
          },
          [&](int row, int sb, int ln, float (&v)[8]) { q4e::load8_f32(p.act, KNJ_DT_F32, (int64_t)row * F + 256 * sb + 8 * ln, v); });
    }
    KNJ_STAMP(6);
    arrivals += G;
    grid_arrive(p.sync);
    if (!grid_wait(p.sync, arrivals, p.wait_cycles)) return;
    KNJ_STAMP(7);

    // ---- stage 5: ordered weighted sum of a token's k rows, residual last, four columns per thread
    {
      const int H4 = H / 4, items = T * H4;
      for (int i = c * kThreads + threadIdx.x; i < items; i += G * kThreads) {
        const int t = i / H4, n = 4 * (i - t * H4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < k; ++s) {
          const int pr = t * k + ord[t * k + s];
          const float w = sel_w[pr];
          const float4 y = __ldcg(reinterpret_cast<const float4 *>(p.Y + (size_t)pr * H + n));
          acc.x = __fadd_rn(acc.x, __fmul_rn(w, y.x));
          acc.y = __fadd_rn(acc.y, __fmul_rn(w, y.y));
          acc.z = __fadd_rn(acc.z, __fmul_rn(w, y.z));
          acc.w = __fadd_rn(acc.w, __fmul_rn(w, y.w));
        }
        if (L.residual) {
          float r[4];
          if (L.x_dtype == KNJ_DT_F32) {
            const float4 xv = __ldcg(reinterpret_cast<const float4 *>(static_cast<const float *>(L.x) + (int64_t)t * L.ldx + n));
            r[0] = xv.x; r[1] = xv.y; r[2] = xv.z; r[3] = xv.w;
          } else {
            const uint2 xv = __ldcg(reinterpret_cast<const uint2 *>(static_cast<const unsigned short *>(L.x) + (int64_t)t * L.ldx + n));
            r[0] = __uint_as_float(xv.x << 16); r[1] = __uint_as_float(xv.x & 0xffff0000u);
            r[2] = __uint_as_float(xv.y << 16); r[3] = __uint_as_float(xv.y & 0xffff0000u);
          }
          acc.x = __fadd_rn(r[0], acc.x); acc.y = __fadd_rn(r[1], acc.y);
          acc.z = __fadd_rn(r[2], acc.z); acc.w = __fadd_rn(r[3], acc.w);
        }
        if (L.out_dtype == KNJ_DT_F32) {
          *reinterpret_cast<float4 *>(static_cast<float *>(L.out) + (int64_t)t * L.ldo + n) = acc;
        } else {
          __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(L.out) + (int64_t)t * L.ldo + n;
          const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
          *reinterpret_cast<uint2 *>(o) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
        }
      }
    }
    KNJ_STAMP(8);
    if (l + 1 < p.n_layers) {
      arrivals += G;
      grid_arrive(p.sync);
      if (!grid_wait(p.sync, arrivals, p.wait_cycles)) return;
    }
    KNJ_STAMP(9);
  }
  if (!ok && threadIdx.x == 0) atomicExch(p.sync + 1, 1u);
}

}  // namespace

namespace {
int g_force_big_stack = 0;  // measurement builds: run the tensor-core kernel for the smallest batches too
}

struct knj_moe_stack {
  SmallStack *small = nullptr;  // batches of at most kSmallStackMaxTokens run the scalar-FMA kernel instead
  StackParams p{};
  void *dev_block = nullptr;  // layer table, logits, scales, activations, per-pair rows, sync words
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
  bool any_q6k = false;  // the scalar kernel of the smallest batches takes Q4_K down matrices only
  for (int l = 0; l < n_layers; ++l) any_q6k = any_q6k || layers[l].down_format == 1;
  if (T <= kSmallStackMaxTokens && !g_force_big_stack && !any_q6k) {
    SmallStack *sm = nullptr;
    const int rc = small_stack_create(layers, n_layers, &sm);
    if (rc) return rc;
    knj_moe_stack *st = new knj_moe_stack();
    st->small = sm;
    *out = st;
    return KNJ_OK;
  }
  KNJ_REQUIRE(H > 0 && H % 256 == 0 && H <= 256 * kMaxSlices, "knj_moe_stack_create: hidden=%d must be a multiple of 256, at most %d", H,
              256 * kMaxSlices);
  KNJ_REQUIRE(F > 0 && F % 256 == 0 && F <= 4096, "knj_moe_stack_create: ffn=%d must be a multiple of 256, at most 4096", F);
  KNJ_REQUIRE(k >= 1 && k <= 8 && k <= E && E <= 256, "knj_moe_stack_create: top_k=%d / n_experts=%d out of range", k, E);
  StackParams sp{};
  sp.gu.N = F; sp.gu.nsb = H / 256; sp.gu.sbs = (sp.gu.nsb % 2 == 0) ? 2 : 1; sp.gu.tiles = F / 8;
  sp.dn.N = H; sp.dn.nsb = F / 256; sp.dn.sbs = (sp.dn.nsb % 2 == 0) ? 2 : 1; sp.dn.tiles = H / 16;
  sp.gu.stages = sp.gu.sbs == 2 ? 2 : q4e::kMaxStages;
  sp.dn.stages = sp.dn.sbs == 2 ? 2 : q4e::kMaxStages;
  std::vector<LayerDesc> table(n_layers);
  std::vector<LayerMaps> maps(n_layers);
  for (int l = 0; l < n_layers; ++l) {
    const knj_moe_ffn_args &a = layers[l];
    KNJ_REQUIRE(a.n_tokens == T && a.hidden == H && a.ffn == F && a.n_experts == E && a.top_k == k,
                "knj_moe_stack_create: layer %d differs in shape from layer 0", l);
    KNJ_REQUIRE(a.x && a.out && a.w_router && a.w_gate && a.w_up && a.w_down, "knj_moe_stack_create: layer %d: null tensor pointer", l);
    KNJ_REQUIRE(a.down_format == 0 || a.down_format == 1, "knj_moe_stack_create: layer %d: unknown format of the down matrices", l);
    KNJ_REQUIRE(a.x_dtype == KNJ_DT_F32 || a.x_dtype == KNJ_DT_BF16, "knj_moe_stack_create: layer %d: x must be f32 or bf16", l);
    KNJ_REQUIRE(a.out_dtype == KNJ_DT_F32 || a.out_dtype == KNJ_DT_BF16, "knj_moe_stack_create: layer %d: out must be f32 or bf16", l);
    KNJ_REQUIRE(a.ldx >= H && a.ldo >= H && a.ldx % 8 == 0 && a.ldo % 4 == 0, "knj_moe_stack_create: layer %d: bad row strides", l);
    auto al16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    KNJ_REQUIRE(al16(a.x) && al16(a.out) && al16(a.w_router) && al16(a.w_gate) && al16(a.w_up) && al16(a.w_down) &&
                    (!a.norm_w || al16(a.norm_w)),
                "knj_moe_stack_create: layer %d: x, out, router, norm and expert bases must be 16-byte aligned", l);
    KNJ_REQUIRE(a.x != a.out, "knj_moe_stack_create: layer %d: out must not alias x (other CTAs still read x)", l);
    LayerDesc &s = table[l];
    LayerMaps &m = maps[l];
    int rc = make_row_tensor_map(&m.mg, a.w_gate, (uint64_t)E * F, (uint32_t)sp.gu.nsb * KNJ_Q4K_BYTES, (uint32_t)sp.gu.sbs * KNJ_Q4K_BYTES, 8);
    if (!rc) rc = make_row_tensor_map(&m.mu, a.w_up, (uint64_t)E * F, (uint32_t)sp.gu.nsb * KNJ_Q4K_BYTES, (uint32_t)sp.gu.sbs * KNJ_Q4K_BYTES, 8);
    if (!rc && a.down_format == 0)
      rc = make_row_tensor_map(&m.md, a.w_down, (uint64_t)E * H, (uint32_t)sp.dn.nsb * KNJ_Q4K_BYTES, (uint32_t)sp.dn.sbs * KNJ_Q4K_BYTES, 16);
    if (rc) return rc;
    s.w_down6 = a.down_format == 1 ? a.w_down : nullptr;
    s.x = a.x;
    s.out = a.out;
    s.Wr = reinterpret_cast<const __nv_bfloat16 *>(a.w_router);
    s.bias = a.router_bias;
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
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    cudaGetLastError();
    set_error("knj_moe_stack_create: the device's properties cannot be read");
    return KNJ_E_RUNTIME;
  }
  // boxes in flight per warp: as many as the shared memory holds next to the panels
  auto total = [&]() { return (size_t)make_plan(sp.gu, sp.dn, T, k).total; };
  while (total() > (size_t)prop.sharedMemPerBlockOptin && (sp.gu.stages > 2 || sp.dn.stages > 2)) {
    if (q4e::phase_ring_bytes(sp.gu.sbs, sp.gu.stages) >= q4e::phase_ring_bytes(sp.dn.sbs, sp.dn.stages) && sp.gu.stages > 2) --sp.gu.stages;
    else if (sp.dn.stages > 2) --sp.dn.stages;
    else --sp.gu.stages;
  }
  const size_t smem = total();
  if (any_q6k) {  // a Q6_K down phase stages a 64-row block and eight activation rows in the ring area
    const size_t need = q6b::block_bytes(F) + q6b::act_scratch_bytes(F, q4e::kWarps);
    const size_t ring = std::max(q4e::phase_ring_bytes(sp.gu.sbs, sp.gu.stages), q4e::phase_ring_bytes(sp.dn.sbs, sp.dn.stages));
    KNJ_REQUIRE(need <= ring, "knj_moe_stack_create: ffn=%d is too long for the Q6_K down phase's staging (%zu > %zu bytes)", F, need, ring);
  }
  if (!prop.cooperativeLaunch || smem > (size_t)prop.sharedMemPerBlockOptin) {
    set_error("knj_moe_stack_create: the device lacks cooperative launch or %zu bytes of shared memory per block", smem);
    return KNJ_E_REFUSE;
  }
  cudaError_t e = cudaFuncSetAttribute(moe_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int per_sm = 0;
  if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_stack_kernel, kThreads, smem);
  if (e != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    set_error("knj_moe_stack_create: the kernel does not fit an SM (%s)", cudaGetErrorString(e));
    return KNJ_E_RUNTIME;
  }
  knj_moe_stack *st = new knj_moe_stack();
  st->device = device;
  st->smem = smem;
  st->grid = sm_count();
  auto up256 = [](size_t n) { return (n + 255) & ~(size_t)255; };
  const size_t P = (size_t)T * k;
  const size_t off_desc = up256((size_t)n_layers * sizeof(LayerMaps));
  const size_t off_logits = off_desc + up256((size_t)n_layers * sizeof(LayerDesc));
  const size_t off_scales = off_logits + up256((size_t)T * E * 4);
  const size_t off_act = off_scales + up256((size_t)T * 4);
  const size_t off_y = off_act + up256(P * F * 4);
  const size_t off_sync = off_y + up256(P * H * 4);
  e = cudaMalloc(&st->dev_block, off_sync + 256);
  if (e == cudaSuccess) e = cudaMemcpy(st->dev_block, maps.data(), (size_t)n_layers * sizeof(LayerMaps), cudaMemcpyHostToDevice);
  if (e == cudaSuccess)
    e = cudaMemcpy(static_cast<char *>(st->dev_block) + off_desc, table.data(), (size_t)n_layers * sizeof(LayerDesc), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (st->dev_block) cudaFree(st->dev_block);
    delete st;
    cudaGetLastError();
    set_error("knj_moe_stack_create: device allocation failed (%s)", cudaGetErrorString(e));
    return KNJ_E_RUNTIME;
  }
  char *base = static_cast<char *>(st->dev_block);
  st->p = sp;
  st->p.maps = reinterpret_cast<const LayerMaps *>(base);
  st->p.layers = reinterpret_cast<const LayerDesc *>(base + off_desc);
  st->p.n_layers = n_layers;
  st->p.T = T; st->p.H = H; st->p.F = F; st->p.E = E; st->p.k = k;
  st->p.logits = reinterpret_cast<float *>(base + off_logits);
  st->p.scales = reinterpret_cast<float *>(base + off_scales);
  st->p.act = reinterpret_cast<float *>(base + off_act);
  st->p.Y = reinterpret_cast<float *>(base + off_y);
  st->p.sync = reinterpret_cast<unsigned int *>(base + off_sync);
  st->p.wait_cycles = kMaxWaitCycles;
  st->p.stall = 0;
  *out = st;
  return KNJ_OK;
}

int knj_moe_stack_decode_launch(knj_moe_stack *st, knj_stream_t s) {
  KNJ_REQUIRE(st && (st->small || st->dev_block), "knj_moe_stack_decode_launch: null stack");
  if (st->small) return small_stack_launch(st->small, s);
  KNJ_CUDA(cudaMemsetAsync(st->p.sync, 0, 8, as_stream(s)));
  void *args[] = {&st->p};
  KNJ_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(moe_stack_kernel), dim3(st->grid), dim3(kThreads), args,
                                       st->smem, as_stream(s)));
  return launch_status("moe_stack_kernel");
}

int knj_moe_stack_set_wait(knj_moe_stack *st, long long wait_cycles, int stall_first_barrier) {
  KNJ_REQUIRE(st, "knj_moe_stack_set_wait: null stack");
  st->p.wait_cycles = wait_cycles > 0 ? wait_cycles : kMaxWaitCycles;
  st->p.stall = stall_first_barrier > 0 ? stall_first_barrier : 0;
  if (st->small) small_stack_set_wait(st->small, st->p.wait_cycles, st->p.stall);
  return KNJ_OK;
}

int knj_moe_stack_status(knj_moe_stack *st, knj_stream_t s) {
  KNJ_REQUIRE(st && (st->small || st->dev_block), "knj_moe_stack_status: null stack");
  if (st->small) return small_stack_status(st->small, s);
  unsigned int words[2] = {0, 0};
  KNJ_CUDA(cudaMemcpyAsync(words, st->p.sync, 8, cudaMemcpyDeviceToHost, as_stream(s)));
  KNJ_CUDA(cudaStreamSynchronize(as_stream(s)));
  if (words[1] != 0) {
    set_error("knj_moe_stack: a bounded wait ran out of time (grid arrivals %u)", words[0]);
    return KNJ_E_TIMEOUT;
  }
  return KNJ_OK;
}

#ifdef KNJ_TRACE
int knj_trace_force_big_stack(int on) { g_force_big_stack = on; return 0; }
int knj_trace_stack(unsigned long long *host_out) {  // measurement build only: 160 CTAs x 16 stamps
  KNJ_CUDA(cudaMemcpyFromSymbol(host_out, g_stack_trace, sizeof(unsigned long long) * 16 * 160));
  return KNJ_OK;
}
#endif

void knj_moe_stack_destroy(knj_moe_stack *st) {
  if (!st) return;
  if (st->small) small_stack_destroy(st->small);
  if (st->dev_block) cudaFree(st->dev_block);
  delete st;
}

}  // extern "C"
