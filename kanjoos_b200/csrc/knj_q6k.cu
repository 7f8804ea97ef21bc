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
#include "knj_q6k_block.cuh"

using namespace knj;

namespace {

constexpr int kQ6Tok = q6b::kTok;     // tokens per pass (accumulators per lane)
constexpr int kQ6Rows = q6b::kRows;   // output rows per work item
constexpr int kQ6Threads = 256;

struct Q6Params {
  const float *A;  // activation rows f32 [P][K]
  const uint8_t *W;  // [E][N][K/256][210]
  const int32_t *pair_idx, *pair_cnt, *exp_list, *n_active;
  float *Y;  // [P][N]
  int N, K;
  int64_t idxStride;
};

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
    const int n0 = chunk * kQ6Rows, n_rows = min(kQ6Rows, p.N - n0);
    __syncthreads();  // the previous item is done with both buffers
    q6b::stage_block(wbuf, p.W + ((size_t)e * p.N + n0) * row_bytes, n_rows * row_bytes, threadIdx.x, kQ6Threads);
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
      q6b::rows_any<kQ6Threads / 32>(wbuf, abuf, p.K, n_rows, nt, lane, warp,
                                     [&](int r, int t, float v) { p.Y[(size_t)s_pair[t] * p.N + n0 + r] = v; });
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
