// knj_q6k.cu -- decode-class projection over Q6_K weights (210-byte superblocks:
// 128 B low nibbles, 64 B high bit pairs, 16 int8 scales, fp16 d;
// w = d * sc * (q - 32)), the format half of the down matrices of Q4_K_M
// checkpoints use. Reference entry point: knj_q6k_down
// (tools/bench/q4k_stream_ffn.hip:780-829) and the CPU dot_q6_k
// (src/loader/dequant.cpp:986-1022).
//
// f32 throughout. A CTA takes (expert, block of up to 64 output rows): the block's superblocks are contiguous in
// HBM and start on a 16-byte boundary every eighth row (rows themselves are only 2-byte aligned, so there are no
// TMA boxes here), and are staged into shared memory with 16-byte loads, once for all of the expert's tokens; the
// activation rows of up to 8 tokens are staged beside them. A warp then walks a row: lane l decodes the four
// weights l, l+32, l+64, l+96 of each 128-weight half (two code bytes, one byte of high bit pairs, four int8
// scales), forms sc * (q - 32) in integers, and feeds one FMA per weight and token; d is applied once per
// superblock, the warp sums meet in shuffles.
#include "knj_common.cuh"
#include "knj_q4k.h"

using namespace knj;

namespace {

constexpr int kQ6Tok = 8;     // tokens per pass (accumulators per lane)
constexpr int kQ6Rows = 64;   // output rows per work item
constexpr int kQ6Threads = 256;

struct Q6Params {
  const float *A;  // activation rows f32 [P][K]
  const uint8_t *W;  // [E][N][K/256][210]
  const int32_t *pair_idx, *pair_cnt, *exp_list, *n_active;
  float *Y;  // [P][N]
  int N, K;
  int64_t idxStride;
};

// four weights of lane `lane` in half `hf` of a superblock, as sc * (q - 32): positions lane, +32, +64, +96
__device__ __forceinline__ void q6k_four(const uint8_t *blk, int hf, int lane, float (&w)[4]) {
  const uint32_t a = blk[64 * hf + lane], b = blk[64 * hf + 32 + lane], h = blk[128 + 32 * hf + lane];
  const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + 8 * hf) + (lane >> 4);
  w[0] = (float)((int)sc[0] * ((int)((a & 15u) | ((h & 3u) << 4)) - 32));
  w[1] = (float)((int)sc[2] * ((int)((b & 15u) | (((h >> 2) & 3u) << 4)) - 32));
  w[2] = (float)((int)sc[4] * ((int)((a >> 4) | (((h >> 4) & 3u) << 4)) - 32));
  w[3] = (float)((int)sc[6] * ((int)((b >> 4) | (((h >> 6) & 3u) << 4)) - 32));
}

// Rows of the staged block against NT staged activation rows: a warp takes rows (r, r + 8) together, so that an
// activation value read from shared memory meets two weights.
template <int NT>
__device__ __forceinline__ void q6k_rows(const Q6Params &p, const uint8_t *wbuf, const float *abuf, const int *s_pair, int n0, int rows,
                                         int nt, int lane, int warp) {
  constexpr int kW = kQ6Threads / 32;
  const int nsb = p.K / KNJ_QK_K, row_bytes = nsb * KNJ_Q6K_BYTES;
  for (int r = warp; r < rows; r += 2 * kW) {
    const bool two = r + kW < rows;
    const int r2 = two ? r + kW : r;
    float acc[2][NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[0][t] = acc[1][t] = 0.f;
    for (int sb = 0; sb < nsb; ++sb) {
      const uint8_t *b0 = wbuf + (size_t)r * row_bytes + sb * KNJ_Q6K_BYTES, *b1 = wbuf + (size_t)r2 * row_bytes + sb * KNJ_Q6K_BYTES;
      float part[2][NT];
#pragma unroll
      for (int t = 0; t < NT; ++t) part[0][t] = part[1][t] = 0.f;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        float w0[4], w1[4];
        q6k_four(b0, hf, lane, w0);
        q6k_four(b1, hf, lane, w1);
        const float *x = abuf + sb * KNJ_QK_K + hf * 128 + lane;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const float *xt = x + (size_t)t * p.K;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float xv = xt[32 * j];
            part[0][t] = fmaf(w0[j], xv, part[0][t]);
            part[1][t] = fmaf(w1[j], xv, part[1][t]);
          }
        }
      }
      const float d0 = knj_half_bits_to_float((uint16_t)(b0[208] | ((uint16_t)b0[209] << 8)));
      const float d1 = knj_half_bits_to_float((uint16_t)(b1[208] | ((uint16_t)b1[209] << 8)));
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        acc[0][t] = fmaf(d0, part[0][t], acc[0][t]);
        acc[1][t] = fmaf(d1, part[1][t], acc[1][t]);
      }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const float v0 = warp_sum(acc[0][t]), v1 = warp_sum(acc[1][t]);
      if (lane == 0 && t < nt) {
        p.Y[(size_t)s_pair[t] * p.N + n0 + r] = v0;
        if (two) p.Y[(size_t)s_pair[t] * p.N + n0 + r2] = v1;
      }
    }
  }
}

__global__ void __launch_bounds__(kQ6Threads) q6k_proj_kernel(const Q6Params p) {
  extern __shared__ __align__(16) uint8_t s_raw[];  // [kQ6Rows][row bytes] weights, then [kQ6Tok][K] f32 activations
  __shared__ int s_pair[kQ6Tok];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nsb = p.K / KNJ_QK_K, row_bytes = nsb * KNJ_Q6K_BYTES;
  uint8_t *wbuf = s_raw;
  float *abuf = reinterpret_cast<float *>(s_raw + (((size_t)kQ6Rows * row_bytes + 15) & ~(size_t)15));
  const int chunks = (p.N + kQ6Rows - 1) / kQ6Rows;
  const int n_act = p.n_active[0];
  const int total = n_act * chunks;
  for (int it = blockIdx.x; it < total; it += gridDim.x) {
    const int a = it / chunks, chunk = it - a * chunks;
    const int e = p.exp_list[a];
    const int cnt = p.pair_cnt[e];
    const int n0 = chunk * kQ6Rows, rows = min(kQ6Rows, p.N - n0);
    __syncthreads();  // the previous item is done with both buffers
    {  // the block's superblocks: contiguous bytes; 16-byte pieces where the start allows it
      const uint8_t *src = p.W + ((size_t)e * p.N + n0) * row_bytes;
      const int bytes = rows * row_bytes;
      if (((reinterpret_cast<uintptr_t>(src) | (uintptr_t)bytes) & 15u) == 0) {
        for (int i = threadIdx.x; i < bytes / 16; i += kQ6Threads)
          reinterpret_cast<uint4 *>(wbuf)[i] = __ldcs(reinterpret_cast<const uint4 *>(src) + i);
      } else {
        for (int i = threadIdx.x; i < bytes / 2; i += kQ6Threads)
          reinterpret_cast<uint16_t *>(wbuf)[i] = reinterpret_cast<const uint16_t *>(src)[i];
      }
    }
    for (int tok0 = 0; tok0 < cnt; tok0 += kQ6Tok) {
      const int nt = min(kQ6Tok, cnt - tok0);
      if (tok0) __syncthreads();  // the previous pass is done with the staged rows
      if ((int)threadIdx.x < kQ6Tok) s_pair[threadIdx.x] = (int)threadIdx.x < nt ? p.pair_idx[(size_t)e * p.idxStride + tok0 + threadIdx.x] : -1;
      __syncthreads();
      for (int i = threadIdx.x; i < nt * (p.K / 4); i += kQ6Threads) {
        const int t = i / (p.K / 4), k4 = i - t * (p.K / 4);
        reinterpret_cast<float4 *>(abuf + (size_t)t * p.K)[k4] = __ldg(reinterpret_cast<const float4 *>(p.A + (size_t)s_pair[t] * p.K) + k4);
      }
      __syncthreads();
      if (nt == 1) q6k_rows<1>(p, wbuf, abuf, s_pair, n0, rows, nt, lane, warp);
      else if (nt == 2) q6k_rows<2>(p, wbuf, abuf, s_pair, n0, rows, nt, lane, warp);
      else if (nt <= 4) {
        for (int i = threadIdx.x; i < (4 - nt) * p.K; i += kQ6Threads) abuf[(size_t)nt * p.K + i] = 0.f;
        __syncthreads();
        q6k_rows<4>(p, wbuf, abuf, s_pair, n0, rows, nt, lane, warp);
      } else {
        for (int i = threadIdx.x; i < (kQ6Tok - nt) * p.K; i += kQ6Threads) abuf[(size_t)nt * p.K + i] = 0.f;
        __syncthreads();
        q6k_rows<kQ6Tok>(p, wbuf, abuf, s_pair, n0, rows, nt, lane, warp);
      }
    }
  }
}

}  // namespace

extern "C" {

int knj_q6k_proj_launch(const float *A, const uint8_t *W6, const int32_t *pair_idx, const int32_t *pair_cnt,
                        const int32_t *exp_list, const int32_t *n_active, float *Y, int N, int K, int64_t idxStride,
                        int n_experts, knj_stream_t s) {
  KNJ_REQUIRE(A && W6 && pair_idx && pair_cnt && exp_list && n_active && Y, "knj_q6k_proj: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && N > 0 && n_experts > 0, "knj_q6k_proj: K=%d must be a multiple of 256, N=%d positive", K, N);
  const size_t row_bytes = (size_t)(K / 256) * KNJ_Q6K_BYTES;
  const size_t smem = ((kQ6Rows * row_bytes + 15) & ~(size_t)15) + (size_t)kQ6Tok * K * sizeof(float);
  KNJ_REQUIRE(smem <= 220 * 1024, "knj_q6k_proj: K=%d is too long for the staged rows", K);
  KNJ_REQUIRE(aligned16(A) && K % 4 == 0, "knj_q6k_proj: activation rows must be 16-byte aligned");
  int dev = 0;
  KNJ_CUDA(cudaGetDevice(&dev));
  static size_t opted[64] = {0};
  if (dev >= 0 && dev < 64 && opted[dev] < smem) {
    KNJ_CUDA(cudaFuncSetAttribute(q6k_proj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KNJ_CUDA(cudaFuncSetAttribute(q6k_proj_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    opted[dev] = smem;
  }
  Q6Params p{A, W6, pair_idx, pair_cnt, exp_list, n_active, Y, N, K, idxStride};
  const long long items = (long long)n_experts * ((N + kQ6Rows - 1) / kQ6Rows);
  const long long cap = (long long)sm_count() * (smem <= 72 * 1024 ? 3 : 1);
  q6k_proj_kernel<<<(unsigned)(items < cap ? items : cap), kQ6Threads, smem, as_stream(s)>>>(p);
  return launch_status("q6k_proj_kernel");
}

}  // extern "C"
