// knj_q4k_mma.cu -- decode-class expert projections: Q4_K weights streamed from
// HBM once, unpacked in registers and multiplied on the fp16 tensor cores as
// EXACT small integers, with the per-32 scale and min applied in f32.
//
// Why this shape. A Q4_K weight costs 0.5625 bytes; at HBM speed one SM must
// consume ~40 weights per clock, which a per-weight convert-and-fma loop on the
// CUDA cores cannot issue. So the 4-bit codes never become floats one by one:
//   * a code q placed in the low mantissa bits of an fp16 word IS the fp16
//     subnormal q * 2^-24 (or q * 2^-20 for a high nibble left in place), so
//     one AND per pair of weights builds a tensor-core A fragment;
//   * activations are split beforehand into a high and a low fp16 plane under a
//     per-vector power-of-two scale (together ~22 significant bits), so the
//     products and the f32 accumulation inside mma.sync are exact to f32 level;
//   * per 32-weight sub-block the integer-valued sum S = sum q*x comes out of
//     two m16n8k16 MMAs and is folded as  acc += (d*sc)*S - (dmin*m)*sum(x),
//     the factored form the reference's CPU decode uses
//     (src/loader/dequant.cpp:954-984 dot_q4_k).
// Weight rows reach shared memory through per-row bulk async copies
// (cp.async.bulk + mbarrier transaction bytes), one copy per lane, into rows
// padded so the fragment loads are bank-conflict free. No dequantised weight is
// ever written anywhere.
//
// Fragment bookkeeping. For one 32-byte code group (64 weights, sub-blocks 2G
// and 2G+1) lane (g = lane/4, t = lane%4) holds bytes 8t..8t+7 of rows g and
// g+8. Word s (s = 0,1) of those feeds MMA step s. Inside a word, bytes 0 and 2
// form the first k-pair and bytes 1 and 3 the second; the activation planes are
// stored with every aligned group of four k permuted to (0,2,1,3) so one
// 16-byte load yields the matching B fragments of both steps.
#include "knj_common.cuh"
#include "knj_q4k.h"

using namespace knj;

namespace {

constexpr int kScalePitch = 18;  // floats per row of the scale table: 8 float2 + 1 pad pair

__host__ __device__ inline size_t panel_vec_bytes(int K) { return (size_t)4 * K + (size_t)K / 8 + 16; }

// ---------------------------------------------------------------------------
// activation prep: x -> (scale, hi plane, lo plane, per-32 sums)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) act_prep_kernel(const void *__restrict__ x, int dtype, int64_t ldx, int K,
                                                       uint8_t *__restrict__ panel) {
  const int v = blockIdx.x;
  const int tid = threadIdx.x;
  const int nquad = K / 4;
  __shared__ float red[4];

  float amax = 0.f;
  for (int q = tid; q < nquad; q += 128)
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(load_as_f32(x, dtype, (int64_t)v * ldx + 4 * q + i)));
  amax = warp_max(amax);
  if ((tid & 31) == 0) red[tid >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));

  // power-of-two scale putting the largest magnitude in [2^13, 2^14)
  int e = 0;
  if (amax > 0.f && amax < 3.0e38f) {
    int ex;
    frexpf(amax, &ex);  // amax = m * 2^ex, m in [0.5, 1)
    e = 14 - ex;
    e = max(-120, min(120, e));
  }
  const float s = ldexpf(1.0f, e);

  uint8_t *base = panel + (size_t)v * panel_vec_bytes(K);
  uint2 *hi = reinterpret_cast<uint2 *>(base);
  uint2 *lo = reinterpret_cast<uint2 *>(base + (size_t)2 * K);
  float *sx = reinterpret_cast<float *>(base + (size_t)4 * K);
  float *inv = reinterpret_cast<float *>(base + (size_t)4 * K + (size_t)K / 8);

  // quads of one 32-wide sub-block sit in 8 consecutive lanes (nquad % 8 == 0, 128 % 8 == 0)
  for (int q = tid; q < nquad; q += 128) {
    float f[4], h[4], l[4];
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[i] = load_as_f32(x, dtype, (int64_t)v * ldx + 4 * q + i) * s;
      const __half hh = __float2half_rn(f[i]);
      h[i] = __half2float(hh);
      const __half ll = __float2half_rn(f[i] - h[i]);
      l[i] = __half2float(ll);
      part += h[i] + l[i];
    }
    // stored order (k0, k2, k1, k3)
    __half2 h01 = __floats2half2_rn(h[0], h[2]), h23 = __floats2half2_rn(h[1], h[3]);
    __half2 l01 = __floats2half2_rn(l[0], l[2]), l23 = __floats2half2_rn(l[1], l[3]);
    hi[q] = make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
    lo[q] = make_uint2(*reinterpret_cast<uint32_t *>(&l01), *reinterpret_cast<uint32_t *>(&l23));
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    if ((tid & 7) == 0) sx[q >> 3] = part;
  }
  if (tid == 0) {
    inv[0] = ldexpf(1.0f, -e);
    inv[1] = inv[2] = inv[3] = 0.f;
  }
}

// ---------------------------------------------------------------------------
// the projection kernel
// ---------------------------------------------------------------------------
struct ProjParams {
  const uint8_t *W0;  // gate (dual) or the single matrix
  const uint8_t *W1;  // up (dual) or null
  const uint8_t *panel;
  const int32_t *pair_idx;
  const int32_t *pair_cnt;
  const int32_t *row_map;  // pair -> panel vector (null: pair / row_div)
  const int32_t *exp_list;
  const int32_t *n_active;
  float *out0;  // dual: G        single: Y
  float *out1;  // dual: U
  float *out2;  // dual: A = silu(G)*U
  int N, K, rowBytes, pitch, row_div, tiles_per_expert;
  int64_t idxStride;
  int *status;  // optional: set to 1 when a bounded wait gave up
};

// DUAL: the m16 tile is 8 gate rows (fragment rows 0..7) + the 8 up rows of the
// same output indices (fragment rows 8..15), so silu(g)*u pairs up in-thread.
// Otherwise the tile is 16 consecutive rows of one matrix.
template <bool DUAL, int NT>
__global__ void __launch_bounds__(512) q4k_proj_kernel(const ProjParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int nsb = p.K / KNJ_QK_K;

  const size_t per_warp = (size_t)16 * p.pitch + 16 * kScalePitch * sizeof(float) + 16;
  uint8_t *wbase = smem + (size_t)warp * per_warp;
  float *scales = reinterpret_cast<float *>(wbase + (size_t)16 * p.pitch);
  uint64_t *bar = reinterpret_cast<uint64_t *>(wbase + (size_t)16 * p.pitch + 16 * kScalePitch * sizeof(float));

  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_init_fence();
  }
  __syncwarp();
  uint32_t phase = 0;

  const int n_act = p.n_active[0];
  const int total = n_act * p.tiles_per_expert;
  const size_t vec_bytes = panel_vec_bytes(p.K);
  const int rows_per_tile = DUAL ? 8 : 16;

  for (int it = blockIdx.x * nwarp + warp; it < total; it += gridDim.x * nwarp) {
    const int a = it / p.tiles_per_expert, tile = it - a * p.tiles_per_expert;
    const int e = p.exp_list[a];
    const int cnt = p.pair_cnt[e];
    const int n0 = tile * rows_per_tile;

    // ---- stream the 16 weight rows of this tile into shared memory
    fence_proxy_async();
    if (lane == 0) mbar_expect_tx(bar, 16u * (uint32_t)p.rowBytes);
    __syncwarp();
    if (lane < 16) {
      const uint8_t *src;
      if (DUAL)
        src = (lane < 8 ? p.W0 : p.W1) + ((size_t)e * p.N + n0 + (lane & 7)) * p.rowBytes;
      else
        src = p.W0 + ((size_t)e * p.N + n0 + lane) * p.rowBytes;
      bulk_g2s(wbase + (size_t)lane * p.pitch, src, (uint32_t)p.rowBytes, bar);
    }
    if (!mbar_wait(bar, phase)) {
      if (lane == 0 && p.status) atomicExch(p.status, 1);
      mbar_wait(bar, phase);  // one more bounded wait for the copies in flight, then leave
      return;
    }
    phase ^= 1u;

    const uint8_t *rowA = wbase + (size_t)g * p.pitch;
    const uint8_t *rowB = wbase + (size_t)(g + 8) * p.pitch;

    for (int tok0 = 0; tok0 < cnt; tok0 += 4 * NT) {
      // pair ids of this token group: lane i holds the pair of token tok0 + i
      int my_pair = -1;
      if (lane < 4 * NT && tok0 + lane < cnt) my_pair = p.pair_idx[(size_t)e * p.idxStride + tok0 + lane];
      int my_vec = -1;
      if (my_pair >= 0) my_vec = p.row_map ? p.row_map[my_pair] : my_pair / p.row_div;

      const uint8_t *bptr[NT];  // B fragments: token g/2 of the tile, plane g&1
      const float *sxptr[NT];   // per-32 sums + inverse scale: token t of the tile
      int out_pair[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int vb = __shfl_sync(0xffffffffu, my_vec, nt * 4 + (g >> 1));
        const int vo = __shfl_sync(0xffffffffu, my_vec, nt * 4 + t);
        out_pair[nt] = __shfl_sync(0xffffffffu, my_pair, nt * 4 + t);
        bptr[nt] = vb >= 0 ? p.panel + (size_t)vb * vec_bytes + (size_t)(g & 1) * 2 * p.K + 16 * t : nullptr;
        sxptr[nt] = vo >= 0 ? reinterpret_cast<const float *>(p.panel + (size_t)vo * vec_bytes + (size_t)4 * p.K)
                            : nullptr;
      }

      float acc0[NT], acc1[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc0[nt] = acc1[nt] = 0.f;

      for (int b = 0; b < nsb; ++b) {
        // ---- (d*sc, dmin*m) of the 16 rows x 8 sub-blocks of this superblock
        __syncwarp();
        if (lane < 16) {
          const uint4 h = *reinterpret_cast<const uint4 *>(wbase + (size_t)lane * p.pitch + (size_t)b * KNJ_Q4K_BYTES);
          const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
          const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
          const uint32_t sc_lo = h.y & 0x3f3f3f3fu, mn_lo = h.z & 0x3f3f3f3fu;
          const uint32_t sc_hi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
          const uint32_t mn_hi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
          float2 *dst = reinterpret_cast<float2 *>(scales + lane * kScalePitch);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t sc = ((j < 4 ? sc_lo : sc_hi) >> (8 * (j & 3))) & 0xffu;
            const uint32_t mn = ((j < 4 ? mn_lo : mn_hi) >> (8 * (j & 3))) & 0xffu;
            // even sub-blocks hold q*2^-24, odd ones q*2^-20
            dst[j] = make_float2(d * (float)sc * ((j & 1) ? 1048576.0f : 16777216.0f), dmin * (float)mn);
          }
        }
        __syncwarp();

        float sx[NT][8];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (sxptr[nt]) {
            const float4 s0 = __ldg(reinterpret_cast<const float4 *>(sxptr[nt] + b * 8));
            const float4 s1 = __ldg(reinterpret_cast<const float4 *>(sxptr[nt] + b * 8 + 4));
            sx[nt][0] = s0.x; sx[nt][1] = s0.y; sx[nt][2] = s0.z; sx[nt][3] = s0.w;
            sx[nt][4] = s1.x; sx[nt][5] = s1.y; sx[nt][6] = s1.z; sx[nt][7] = s1.w;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) sx[nt][j] = 0.f;
          }
        }

#pragma unroll
        for (int G = 0; G < 4; ++G) {
          const size_t off = (size_t)b * KNJ_Q4K_BYTES + KNJ_Q4K_OFF_QS + 32 * G + 8 * t;
          const uint2 wa = *reinterpret_cast<const uint2 *>(rowA + off);
          const uint2 wb = *reinterpret_cast<const uint2 *>(rowB + off);
#pragma unroll
          for (int par = 0; par < 2; ++par) {
            const int j = 2 * G + par;
            const uint32_t M = par ? 0x00f000f0u : 0x000f000fu;
            const float2 sa = *reinterpret_cast<const float2 *>(scales + g * kScalePitch + 2 * j);
            const float2 sb = *reinterpret_cast<const float2 *>(scales + (g + 8) * kScalePitch + 2 * j);
            const uint32_t a00 = wa.x & M, a01 = wb.x & M, a02 = (wa.x >> 8) & M, a03 = (wb.x >> 8) & M;
            const uint32_t a10 = wa.y & M, a11 = wb.y & M, a12 = (wa.y >> 8) & M, a13 = (wb.y >> 8) & M;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              uint4 bf = make_uint4(0u, 0u, 0u, 0u);
              if (bptr[nt]) bf = __ldg(reinterpret_cast<const uint4 *>(bptr[nt] + (size_t)(b * 256 + 64 * G + 32 * par) * 2));
              float c[4] = {0.f, 0.f, 0.f, 0.f};
              mma_f16_16816(c, a00, a01, a02, a03, bf.x, bf.y);
              mma_f16_16816(c, a10, a11, a12, a13, bf.z, bf.w);
              // columns 2t / 2t+1 are the high / low plane of the same token
              acc0[nt] = fmaf(sa.x, c[0] + c[1], acc0[nt]);
              acc0[nt] = fmaf(-sa.y, sx[nt][j], acc0[nt]);
              acc1[nt] = fmaf(sb.x, c[2] + c[3], acc1[nt]);
              acc1[nt] = fmaf(-sb.y, sx[nt][j], acc1[nt]);
            }
          }
        }
      }

      // ---- epilogue: undo the activation scale, store
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int pp = out_pair[nt];
        if (pp < 0) continue;
        const float inv = __ldg(sxptr[nt] + p.K / 32);
        const float v0 = acc0[nt] * inv, v1 = acc1[nt] * inv;
        if (DUAL) {
          const size_t o = (size_t)pp * p.N + n0 + g;
          if (p.out0) p.out0[o] = v0;
          if (p.out1) p.out1[o] = v1;
          if (p.out2) p.out2[o] = (v0 / (1.0f + expf(-v0))) * v1;
        } else {
          p.out0[(size_t)pp * p.N + n0 + g] = v0;
          p.out0[(size_t)pp * p.N + n0 + g + 8] = v1;
        }
      }
    }
    __syncwarp();
  }
}

__global__ void iota_plan_kernel(int32_t *pair_idx, int32_t *pair_cnt, int32_t *exp_list, int32_t *n_active, int m) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < m) pair_idx[i] = i;
  if (i == 0) {
    pair_cnt[0] = m;
    exp_list[0] = 0;
    n_active[0] = 1;
    n_active[1] = m;
  }
}

int pad_pitch(int rowBytes) {
  int pitch = rowBytes;
  while ((pitch % 128) != 32 && (pitch % 128) != 96) pitch += 16;
  return pitch;
}

template <bool DUAL, int NT>
int launch_proj(const ProjParams &p, int n_experts_max, cudaStream_t st) {
  const size_t per_warp = (size_t)16 * p.pitch + 16 * kScalePitch * sizeof(float) + 16;
  int dev = 0;
  KNJ_CUDA(cudaGetDevice(&dev));
  int smem_max = 0;
  KNJ_CUDA(cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  int warps = (int)((size_t)(smem_max - 1024) / per_warp);
  if (warps > 16) warps = 16;
  KNJ_REQUIRE(warps >= 1, "q4k projection: a %d-byte row does not fit the shared memory tile", p.rowBytes);
  const size_t smem = per_warp * warps;
  auto kern = q4k_proj_kernel<DUAL, NT>;
  // opt in to the large dynamic shared memory once per device and instantiation
  // (kept out of later launches so they are plain stream work, capturable in a graph)
  static size_t opted[64] = {0};
  if (dev >= 0 && dev < 64 && opted[dev] < smem) {
    KNJ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    opted[dev] = smem;
  }
  const long long max_items = (long long)n_experts_max * p.tiles_per_expert;
  long long grid = (max_items + warps - 1) / warps;
  const long long cap = (long long)sm_count();
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  kern<<<(unsigned)grid, warps * 32, smem, st>>>(p);
  return launch_status("q4k_proj_kernel");
}

template <bool DUAL>
int launch_proj_nt(const ProjParams &p, int n_experts_max, int max_tokens, cudaStream_t st) {
  if (max_tokens <= 4) return launch_proj<DUAL, 1>(p, n_experts_max, st);
  if (max_tokens <= 8) return launch_proj<DUAL, 2>(p, n_experts_max, st);
  return launch_proj<DUAL, 4>(p, n_experts_max, st);
}

}  // namespace

extern "C" {

size_t knj_panel_bytes(int n_vec, int K) { return (size_t)(n_vec > 0 ? n_vec : 0) * panel_vec_bytes(K); }

int knj_act_prep_launch(const void *x, int x_dtype, int64_t ldx, int n_vec, int K, void *panel, knj_stream_t s) {
  KNJ_REQUIRE(x && panel, "knj_act_prep: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0, "knj_act_prep: K=%d must be a multiple of 256", K);
  KNJ_REQUIRE(x_dtype >= KNJ_DT_F32 && x_dtype <= KNJ_DT_F16, "knj_act_prep: unknown dtype %d", x_dtype);
  KNJ_REQUIRE(aligned16(panel), "knj_act_prep: panel must be 16-byte aligned");
  if (n_vec <= 0) return KNJ_OK;
  act_prep_kernel<<<n_vec, 128, 0, as_stream(s)>>>(x, x_dtype, ldx, K, static_cast<uint8_t *>(panel));
  return launch_status("act_prep_kernel");
}

int knj_q4k_gateup_launch(const void *Xpanel, const uint8_t *Wg, const uint8_t *Wu, const int32_t *pair_idx,
                          const int32_t *pair_cnt, const int32_t *pair_tok, const int32_t *exp_list,
                          const int32_t *n_active, float *G, float *U, float *A, int N, int K, int rowBytes,
                          int64_t idxStride, int n_experts, int top_k, int max_tokens, knj_stream_t s) {
  KNJ_REQUIRE(Xpanel && Wg && Wu && pair_idx && pair_cnt && exp_list && n_active, "knj_q4k_gateup: null pointer");
  KNJ_REQUIRE(G || U || A, "knj_q4k_gateup: no output requested");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES,
              "knj_q4k_gateup: rowBytes=%d does not match K=%d", rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % 8 == 0, "knj_q4k_gateup: N=%d must be a multiple of 8", N);
  KNJ_REQUIRE(aligned16(Wg) && aligned16(Wu) && aligned16(Xpanel), "knj_q4k_gateup: weights/panel must be 16-byte aligned");
  KNJ_REQUIRE(n_experts > 0 && (pair_tok || top_k > 0), "knj_q4k_gateup: bad expert / top_k count");
  ProjParams p{};
  p.W0 = Wg; p.W1 = Wu; p.panel = static_cast<const uint8_t *>(Xpanel);
  p.pair_idx = pair_idx; p.pair_cnt = pair_cnt; p.row_map = pair_tok; p.exp_list = exp_list; p.n_active = n_active;
  p.out0 = G; p.out1 = U; p.out2 = A;
  p.N = N; p.K = K; p.rowBytes = rowBytes; p.pitch = pad_pitch(rowBytes); p.row_div = top_k > 0 ? top_k : 1;
  p.tiles_per_expert = N / 8; p.idxStride = idxStride; p.status = nullptr;
  return launch_proj_nt<true>(p, n_experts, max_tokens, as_stream(s));
}

int knj_q4k_proj_launch(const void *Apanel, const uint8_t *W, const int32_t *pair_idx, const int32_t *pair_cnt,
                        const int32_t *pair_row, const int32_t *exp_list, const int32_t *n_active, float *Y, int N,
                        int K, int rowBytes, int64_t idxStride, int n_experts, int max_tokens, knj_stream_t s) {
  KNJ_REQUIRE(Apanel && W && pair_idx && pair_cnt && exp_list && n_active && Y, "knj_q4k_proj: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES,
              "knj_q4k_proj: rowBytes=%d does not match K=%d", rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % 16 == 0, "knj_q4k_proj: N=%d must be a multiple of 16", N);
  KNJ_REQUIRE(aligned16(W) && aligned16(Apanel), "knj_q4k_proj: weights/panel must be 16-byte aligned");
  KNJ_REQUIRE(n_experts > 0, "knj_q4k_proj: bad expert count");
  ProjParams p{};
  p.W0 = W; p.W1 = nullptr; p.panel = static_cast<const uint8_t *>(Apanel);
  p.pair_idx = pair_idx; p.pair_cnt = pair_cnt; p.row_map = pair_row; p.exp_list = exp_list; p.n_active = n_active;
  p.out0 = Y; p.out1 = nullptr; p.out2 = nullptr;
  p.N = N; p.K = K; p.rowBytes = rowBytes; p.pitch = pad_pitch(rowBytes); p.row_div = 1;
  p.tiles_per_expert = N / 16; p.idxStride = idxStride; p.status = nullptr;
  return launch_proj_nt<false>(p, n_experts, max_tokens, as_stream(s));
}

size_t knj_q4k_matmul_workspace_bytes(int m, int n_in) {
  if (m <= 0 || n_in <= 0) return 0;
  // panel + identity pair list + counts
  return ((knj_panel_bytes(m, n_in) + 255) & ~(size_t)255) + (((size_t)m * 4 + 255) & ~(size_t)255) + 256;
}

int knj_q4k_matmul_launch(const uint8_t *W, int n_in, int n_out, const void *x, int x_dtype, int64_t ldx, int m,
                          float *y, int64_t ldy, void *workspace, size_t workspace_bytes, knj_stream_t s) {
  KNJ_REQUIRE(W && x && y, "knj_q4k_matmul: null pointer");
  KNJ_REQUIRE(m > 0 && n_in % 256 == 0 && n_out % 16 == 0, "knj_q4k_matmul: needs n_in %% 256 == 0, n_out %% 16 == 0");
  KNJ_REQUIRE(ldy == n_out, "knj_q4k_matmul: y must be dense (ldy == n_out)");
  if (!workspace || workspace_bytes < knj_q4k_matmul_workspace_bytes(m, n_in)) {
    set_error("knj_q4k_matmul: workspace of %zu bytes needed", knj_q4k_matmul_workspace_bytes(m, n_in));
    return KNJ_E_WORKSPACE;
  }
  KNJ_REQUIRE(aligned16(workspace), "knj_q4k_matmul: workspace must be 16-byte aligned");
  uint8_t *ws = static_cast<uint8_t *>(workspace);
  void *panel = ws;
  ws += (knj_panel_bytes(m, n_in) + 255) & ~(size_t)255;
  int32_t *pair_idx = reinterpret_cast<int32_t *>(ws);
  ws += ((size_t)m * 4 + 255) & ~(size_t)255;
  int32_t *small = reinterpret_cast<int32_t *>(ws);  // [0] cnt, [1] exp_list, [2..3] n_active
  int rc = knj_act_prep_launch(x, x_dtype, ldx, m, n_in, panel, s);
  if (rc) return rc;
  iota_plan_kernel<<<(m + 255) / 256, 256, 0, as_stream(s)>>>(pair_idx, small + 0, small + 1, small + 2, m);
  rc = launch_status("iota_plan_kernel");
  if (rc) return rc;
  return knj_q4k_proj_launch(panel, W, pair_idx, small + 0, nullptr, small + 1, small + 2, y, n_out, n_in,
                             n_in / 256 * KNJ_Q4K_BYTES, m, 1, m, s);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of knj_q4k_matmul_launch.
//
// Who needs it: callers that must not allocate device memory at the point of
// the call and have no workspace to hand over -- code running inside a
// latency-critical serving loop whose memory pool is fully committed to the
// resident experts, plug-in hosts that are only given the input and output
// buffers, and callers that forbid allocator calls after start-up because an
// allocation can synchronise the device or fragment a tightly packed HBM budget.
// For them the scratch lives in a fixed array inside the library image.
//
// Cost and limits: every GPU that loads the library carries the array
// (kNoAllocScratchBytes) until the process exits. Problems whose scratch need
// exceeds it are refused with KNJ_E_WORKSPACE. All calls on a device share the
// one array and it keeps whatever the previous call left there; this entry
// point rewrites every byte it later reads, so nothing needs clearing, but two
// calls whose kernels overlap on the GPU (different streams, or one stream per
// thread) race on it -- serialise them.
//
// The first call on each device resolves the array's device address (the name
// of a __device__ array is only a host-side handle in host code; kernels must be
// given the address cudaGetSymbolAddress returns). Make that first call before
// starting any stream capture.
// ---------------------------------------------------------------------------
namespace {
constexpr size_t kNoAllocScratchBytes = (size_t)1 << 20;  // 1 MiB
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

int noalloc_scratch_ptr(void **out) {
  static void *resolved[64] = {nullptr};
  int dev = 0;
  KNJ_CUDA(cudaGetDevice(&dev));
  KNJ_REQUIRE(dev >= 0 && dev < 64, "no-alloc scratch: device index %d out of range", dev);
  if (!resolved[dev]) {
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);  // with `dev` current
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
    KNJ_REQUIRE(ptr != nullptr, "no-alloc scratch: symbol address resolved to null");
    resolved[dev] = ptr;
  }
  *out = resolved[dev];
  return KNJ_OK;
}
}  // namespace

size_t knj_q4k_matmul_noalloc_max_scratch(void) { return kNoAllocScratchBytes; }

int knj_q4k_matmul_noalloc_launch(const uint8_t *W, int n_in, int n_out, const void *x, int x_dtype, int64_t ldx, int m,
                                  float *y, int64_t ldy, knj_stream_t s) {
  KNJ_REQUIRE(m > 0 && n_in > 0, "knj_q4k_matmul_noalloc: m and n_in must be positive");
  const size_t need = knj_q4k_matmul_workspace_bytes(m, n_in);
  if (need > kNoAllocScratchBytes) {
    set_error("knj_q4k_matmul_noalloc: m=%d rows of n_in=%d need %zu bytes of scratch, the built-in array holds %zu; "
              "use knj_q4k_matmul_launch with a caller workspace",
              m, n_in, need, kNoAllocScratchBytes);
    return KNJ_E_WORKSPACE;
  }
  void *scratch = nullptr;
  int rc = noalloc_scratch_ptr(&scratch);
  if (rc) return rc;
  return knj_q4k_matmul_launch(W, n_in, n_out, x, x_dtype, ldx, m, y, ldy, scratch, kNoAllocScratchBytes, s);
}

}  // extern "C"
