// knj_ep.cu -- kernels around the expert-parallel exchange: rows are packed in
// (destination rank, expert, pair) order before the dispatch all-to-all, and the
// receiving rank turns the per-source expert counts into its local grouped-GEMM
// plan. The reference has no multi-GPU path (it keeps every expert on one
// device: docs/01-architecture.md:322-325); these entry points serve the
// expert-sharded layout this library adds, and follow the pair/plan conventions
// of the single-device path (tools/bench/q4k_stream_ffn.hip:957-1001).
#include "knj_common.cuh"

using namespace knj;

namespace {

// send_off[e] = number of pairs routed to experts < e (exclusive scan of
// pair_cnt), one CTA. E <= 256.
__global__ void __launch_bounds__(256) ep_offsets_kernel(const int32_t *__restrict__ pair_cnt, int E,
                                                         int32_t *__restrict__ send_off) {
  __shared__ int s[256];
  const int e = threadIdx.x;
  s[e] = e < E ? pair_cnt[e] : 0;
  __syncthreads();
  if (e == 0) {
    int run = 0;
    for (int i = 0; i < E; ++i) { const int c = s[i]; s[i] = run; run += c; }
    send_off[E] = run;
  }
  __syncthreads();
  if (e < E) send_off[e] = s[e];
}

// One CTA per send slot group: copies the hidden row of every pair into the
// send buffer in expert-major order and records where each pair went.
__global__ void __launch_bounds__(256) ep_pack_kernel(const uint4 *__restrict__ x, int64_t row_u4, int top_k,
                                                      const int32_t *__restrict__ pair_idx, int idx_stride,
                                                      const int32_t *__restrict__ pair_cnt,
                                                      const int32_t *__restrict__ send_off, int E,
                                                      uint4 *__restrict__ send_rows, int32_t *__restrict__ pair_row) {
  const int e = blockIdx.y;
  const int cnt = pair_cnt[e];
  const int base = send_off[e];
  for (int i = blockIdx.x; i < cnt; i += gridDim.x) {
    const int p = pair_idx[(size_t)e * idx_stride + i];
    const uint4 *src = x + (size_t)(p / top_k) * row_u4;
    uint4 *dst = send_rows + (size_t)(base + i) * row_u4;
    for (int j = threadIdx.x; j < row_u4; j += 256) dst[j] = __ldg(src + j);
    if (threadIdx.x == 0) pair_row[p] = base + i;
  }
}

// Local plan of the receiving rank. counts[r][e] = rows rank r sends for my
// local expert e; rows from rank r arrive contiguously, experts ascending. One
// CTA per local expert lists its rows (source ranks in ascending order).
__global__ void __launch_bounds__(256) ep_plan_kernel(const int32_t *__restrict__ counts, int G, int E_loc,
                                                      int idx_stride, int32_t *__restrict__ pair_idx,
                                                      int32_t *__restrict__ pair_cnt) {
  const int e = blockIdx.x;
  __shared__ int src_base[64];  // first received row of (rank r, expert e)
  __shared__ int dst_base[65];
  if (threadIdx.x == 0) {
    int row = 0, mine = 0;
    for (int r = 0; r < G; ++r) {
      int before = 0, all = 0;
      for (int j = 0; j < E_loc; ++j) {
        const int c = counts[r * E_loc + j];
        if (j < e) before += c;
        all += c;
      }
      src_base[r] = row + before;
      dst_base[r] = mine;
      mine += counts[r * E_loc + e];
      row += all;
    }
    dst_base[G] = mine;
  }
  __syncthreads();
  int32_t *out = pair_idx + (size_t)e * idx_stride;
  const int total = min(dst_base[G], idx_stride);
  for (int r = 0; r < G; ++r) {
    const int c = dst_base[r + 1] - dst_base[r];
    for (int i = threadIdx.x; i < c; i += 256)
      if (dst_base[r] + i < idx_stride) out[dst_base[r] + i] = src_base[r] + i;
  }
  for (int i = total + threadIdx.x; i < idx_stride; i += 256) out[i] = -1;
  if (threadIdx.x == 0) pair_cnt[e] = total;
}

}  // namespace

extern "C" {

int knj_ep_pack_launch(const void *x, int row_bytes, int top_k, const int32_t *pair_idx, int idx_stride,
                       const int32_t *pair_cnt, int E, int32_t *send_off, void *send_rows, int32_t *pair_row,
                       knj_stream_t s) {
  KNJ_REQUIRE(x && pair_idx && pair_cnt && send_off && send_rows && pair_row, "knj_ep_pack: null pointer");
  KNJ_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && aligned16(x) && aligned16(send_rows),
              "knj_ep_pack: rows must be 16-byte multiples at 16-byte aligned bases");
  KNJ_REQUIRE(E >= 1 && E <= 256 && top_k >= 1, "knj_ep_pack: bad expert count / top_k");
  ep_offsets_kernel<<<1, 256, 0, as_stream(s)>>>(pair_cnt, E, send_off);
  int rc = launch_status("ep_offsets_kernel");
  if (rc) return rc;
  dim3 grid(64, E);
  ep_pack_kernel<<<grid, 256, 0, as_stream(s)>>>(static_cast<const uint4 *>(x), row_bytes / 16, top_k, pair_idx,
                                                 idx_stride, pair_cnt, send_off, E, static_cast<uint4 *>(send_rows),
                                                 pair_row);
  return launch_status("ep_pack_kernel");
}

int knj_ep_plan_launch(const int32_t *counts, int n_ranks, int n_local_experts, int idx_stride, int32_t *pair_idx,
                       int32_t *pair_cnt, int32_t *exp_list, int32_t *n_active, knj_stream_t s) {
  KNJ_REQUIRE(counts && pair_idx && pair_cnt && exp_list && n_active, "knj_ep_plan: null pointer");
  KNJ_REQUIRE(n_ranks >= 1 && n_ranks <= 64 && n_local_experts >= 1 && idx_stride >= 1, "knj_ep_plan: bad sizes");
  ep_plan_kernel<<<n_local_experts, 256, 0, as_stream(s)>>>(counts, n_ranks, n_local_experts, idx_stride, pair_idx,
                                                            pair_cnt);
  int rc = launch_status("ep_plan_kernel");
  if (rc) return rc;
  return knj_active_list_launch(pair_cnt, n_local_experts, exp_list, n_active, s);
}

}  // extern "C"
