// knj_q6k.cu -- decode-class projection over Q6_K weights (210-byte superblocks:
// 128 B low nibbles, 64 B high bit pairs, 16 int8 scales, fp16 d;
// w = d * sc * (q - 32)), the format half of the down matrices of Q4_K_M
// checkpoints use. Reference entry point: knj_q6k_down
// (tools/bench/q4k_stream_ffn.hip:780-829) and the CPU dot_q6_k
// (src/loader/dequant.cpp:986-1022).
//
// First correct version, f32 throughout and not tuned: one warp per output row,
// lanes take the row's 16-weight spans (one int8 scale each), decode them with
// knj_q6k_span16 straight from global memory (rows are only 2-byte aligned, so
// there is no bulk-copy staging), multiply with the staged activation rows of up
// to 8 tokens of the expert and reduce over the warp with shuffles.
#include "knj_common.cuh"
#include "knj_q4k.h"

using namespace knj;

namespace {

constexpr int kQ6Tok = 8;     // tokens per pass (accumulators per lane)
constexpr int kQ6Rows = 64;   // output rows per work item

struct Q6Params {
  const float *A;  // activation rows f32 [P][K]
  const uint8_t *W;  // [E][N][K/256][210]
  const int32_t *pair_idx, *pair_cnt, *exp_list, *n_active;
  float *Y;  // [P][N]
  int N, K;
  int64_t idxStride;
};

__global__ void __launch_bounds__(256) q6k_proj_kernel(const Q6Params p) {
  extern __shared__ float s_act[];  // [kQ6Tok][K]
  __shared__ int s_pair[kQ6Tok];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nblk = p.K / KNJ_QK_K, nspan = p.K / 16;
  const int chunks = (p.N + kQ6Rows - 1) / kQ6Rows;
  const int n_act = p.n_active[0];
  const int total = n_act * chunks;
  for (int it = blockIdx.x; it < total; it += gridDim.x) {
    const int a = it / chunks, chunk = it - a * chunks;
    const int e = p.exp_list[a];
    const int cnt = p.pair_cnt[e];
    for (int tok0 = 0; tok0 < cnt; tok0 += kQ6Tok) {
      const int nt = min(kQ6Tok, cnt - tok0);
      __syncthreads();  // the previous pass is done with the staged rows
      if ((int)threadIdx.x < kQ6Tok) s_pair[threadIdx.x] = (int)threadIdx.x < nt ? p.pair_idx[(size_t)e * p.idxStride + tok0 + threadIdx.x] : -1;
      __syncthreads();
      for (int i = threadIdx.x; i < kQ6Tok * p.K; i += 256) {
        const int t = i / p.K, k = i - t * p.K;
        s_act[i] = t < nt ? p.A[(size_t)s_pair[t] * p.K + k] : 0.f;
      }
      __syncthreads();
      for (int r = warp; r < kQ6Rows; r += 8) {
        const int n = chunk * kQ6Rows + r;
        if (n >= p.N) break;
        const uint8_t *row = p.W + ((size_t)e * p.N + n) * nblk * KNJ_Q6K_BYTES;
        float acc[kQ6Tok];
#pragma unroll
        for (int t = 0; t < kQ6Tok; ++t) acc[t] = 0.f;
        for (int sp = lane; sp < nspan; sp += 32) {
          float w[16];
          knj_q6k_span16(row + (size_t)(sp >> 4) * KNJ_Q6K_BYTES, (sp & 15) * 16, w);
#pragma unroll
          for (int t = 0; t < kQ6Tok; ++t) {
            const float *x = s_act + t * p.K + sp * 16;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) sum = fmaf(w[i], x[i], sum);
            acc[t] += sum;
          }
        }
#pragma unroll
        for (int t = 0; t < kQ6Tok; ++t) {
          const float v = warp_sum(acc[t]);
          if (lane == 0 && t < nt) p.Y[(size_t)s_pair[t] * p.N + n] = v;
        }
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
  const size_t smem = (size_t)kQ6Tok * K * sizeof(float);
  KNJ_REQUIRE(smem <= 200 * 1024, "knj_q6k_proj: K=%d is too long for the staged activation rows", K);
  int dev = 0;
  KNJ_CUDA(cudaGetDevice(&dev));
  static size_t opted[64] = {0};
  if (dev >= 0 && dev < 64 && opted[dev] < smem) {
    KNJ_CUDA(cudaFuncSetAttribute(q6k_proj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    opted[dev] = smem;
  }
  Q6Params p{A, W6, pair_idx, pair_cnt, exp_list, n_active, Y, N, K, idxStride};
  const long long items = (long long)n_experts * ((N + kQ6Rows - 1) / kQ6Rows);
  const long long cap = (long long)sm_count() * 4;
  q6k_proj_kernel<<<(unsigned)(items < cap ? items : cap), 256, smem, as_stream(s)>>>(p);
  return launch_status("q6k_proj_kernel");
}

}  // extern "C"
