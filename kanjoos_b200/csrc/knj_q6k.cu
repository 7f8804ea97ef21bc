// knj_q6k.cu -- decode-class projection over Q6_K weights (210-byte superblocks:
// 128 B low nibbles, 64 B high bit pairs, 16 int8 scales, fp16 d;
// w = d * sc * (q - 32)), the format half of the down matrices of Q4_K_M
// checkpoints use. Reference entry point: knj_q6k_down
// (tools/bench/q4k_stream_ffn.hip:780-829) and the CPU dot_q6_k
// (src/loader/dequant.cpp:986-1022).
//
// A CTA takes (expert, block of 64 output rows): a block's superblocks are contiguous in HBM and start
// on a 16-byte boundary (rows themselves are only 2-byte aligned, so there are no TMA boxes here); they travel as one
// bulk copy per block while the CTA prepares the activation side of up to 8 of the expert's tokens (two CTAs per SM:
// one's block travels while the other computes). The block then runs on mma.sync.m16n8k16: one k-step per
// 16-weight scale group, the codes as exact fp16 integers, the activations as two fp16 planes (f32-level accuracy:
// knj_q6k_block.cuh). A scalar form (one FMA per weight and token on integer sc * (q - 32)) was the first version
// and measured slower at every batch, one-token experts included.
#include "knj_common.cuh"
#include "knj_q4k.h"
#include "knj_q6k_block.cuh"

using namespace knj;

namespace {

constexpr int kQ6Tok = q6b::kTok;     // tokens per pass
constexpr int kQ6Rows = q6b::kRows;   // output rows per staged block
constexpr int kQ6MaxSub = 1;          // blocks per work item (the activation side is prepared once per item): with two CTAs
                                      // per SM two or four blocks per item measured no faster (118 us at batch 64 either way)
constexpr int kQ6Threads = 256;  // two CTAs per SM: one's block travels while the other computes

struct Q6Params {
  const float *A;  // activation rows f32 [P][K]
  const uint8_t *W;  // [E][N][K/256][210]
  const int32_t *pair_idx, *pair_cnt, *exp_list, *n_active;
  float *Y;  // [P][N]
  int N, K;
  int64_t idxStride;
  int *status;  // raised when the bounded wait for a weight block gave up (may be null)
  long long wait_cycles;
  int two_blocks;  // the shared memory holds two weight blocks (the next one travels while this one is worked on)
};

__global__ void __launch_bounds__(kQ6Threads, 2) q6k_proj_kernel(const Q6Params p) {
  extern __shared__ __align__(16) uint8_t s_raw[];  // weight block(s), then the activation side (q6b::carve)
  __shared__ int s_pair[kQ6Tok];
  __shared__ uint64_t s_bars[2];  // the weight blocks' bulk copies
  __shared__ int s_fail;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(&s_bars[0], 1);
    mbar_init(&s_bars[1], 1);
    s_fail = 0;
    mbar_init_fence();
  }
  const int row_bytes = p.K / KNJ_QK_K * KNJ_Q6K_BYTES;
  const q6b::Bufs b = q6b::carve(s_raw, p.K, kQ6Threads / 32, p.two_blocks != 0, s_bars, &s_fail);
  const int blocks = (p.N + kQ6Rows - 1) / kQ6Rows;
  const int n_act = p.n_active[0];
  // blocks per item: as many as leave every CTA about two items (few experts: one block per item)
  const int sub = max(1, min(kQ6MaxSub, n_act * blocks / (2 * (int)gridDim.x)));
  const int chunks = (blocks + sub - 1) / sub;
  const int total = n_act * chunks;
  const bool bulk = (reinterpret_cast<uintptr_t>(p.W) & 15u) == 0 && p.N % kQ6Rows == 0;
  unsigned staged = 0;  // bulk copies waited for so far
  for (int it = blockIdx.x; it < total; it += gridDim.x) {
    const int a = it / chunks, chunk = it - a * chunks;
    const int e = p.exp_list[a];
    const int cnt = p.pair_cnt[e];
    const int n0 = chunk * sub * kQ6Rows, n_rows = min(sub * kQ6Rows, p.N - n0);
    for (int tok0 = 0; tok0 < cnt; tok0 += kQ6Tok) {
      const int nt = min(kQ6Tok, cnt - tok0);
      __syncthreads();  // the previous pass is done with the shared buffers
      if ((int)threadIdx.x < kQ6Tok) s_pair[threadIdx.x] = (int)threadIdx.x < nt ? p.pair_idx[(size_t)e * p.idxStride + tok0 + threadIdx.x] : -1;
      __syncthreads();
      if (!q6b::chunk_pass<kQ6Threads / 32>(b, p.W + ((size_t)e * p.N + n0) * row_bytes, n_rows, p.K, p.A, p.Y + n0, p.N, s_pair, nt, staged,
                                            bulk, p.wait_cycles, lane, warp)) {
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, 1);  // a copy that never completed: report and leave
        return;
      }
    }
  }
}

}  // namespace

extern "C" {

int knj_q6k_proj_launch(const float *A, const uint8_t *W6, const int32_t *pair_idx, const int32_t *pair_cnt,
                        const int32_t *exp_list, const int32_t *n_active, float *Y, int N, int K, int64_t idxStride,
                        int n_experts, int *status, knj_stream_t s) {
  KNJ_REQUIRE(A && W6 && pair_idx && pair_cnt && exp_list && n_active && Y, "knj_q6k_proj: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && N > 0 && n_experts > 0, "knj_q6k_proj: K=%d must be a multiple of 256, N=%d positive", K, N);
  const size_t one = q6b::block_bytes(K) + q6b::act_scratch_bytes(K, kQ6Threads / 32);
  const bool two = false;  // one block buffer per CTA and two CTAs per SM measured faster than one CTA with two buffers
  const size_t smem = one + (two ? q6b::block_bytes(K) : 0);
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
  Q6Params p{A, W6, pair_idx, pair_cnt, exp_list, n_active, Y, N, K, idxStride, status, knj::decode_wait_cycles(), two ? 1 : 0};
  const long long items = (long long)n_experts * ((N + kQ6Rows - 1) / kQ6Rows);
  const long long per_sm = smem + 1024 <= 113 * 1024 ? 2 : 1;
  const long long cap = (long long)sm_count() * per_sm;
  q6k_proj_kernel<<<(unsigned)(items < cap ? items : cap), kQ6Threads, smem, as_stream(s)>>>(p);
  return launch_status("q6k_proj_kernel");
}

}  // extern "C"
