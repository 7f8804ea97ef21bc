// knj_q4k_mma.cu -- decode-class expert projections as stand-alone launches:
// gate+up+SiLU*up (tools/bench/q4k_moe_ffn.hip:164-241 knj_q4k_gateup fused with
// tools/bench/q4k_stream_ffn.hip:1021-1031), the single-matrix projection
// (tools/bench/q4k_stream_ffn.hip:834-882 knj_q4k_proj) and Model::matmul
// (src/model/model.cpp:326-380), all on the tile engine of knj_q4k_engine.cuh.
//
// One persistent CTA per SM, 16 warps in teams of `ks` = K / 256 warps. The work
// of a launch is the flat list (job, tile): a JOB is one active expert with up to
// 8 of its tokens (an expert with more tokens yields several jobs; its weights
// then come from L2 after the first), a tile is 16 weight rows. Every team takes
// an equal contiguous run of that list. Each warp runs its own ring of TMA boxes
// (16 rows x 144 bytes: its superblock column of a tile), filled `stages` tiles
// ahead and across job boundaries, so the weight stream never waits for the
// arithmetic; the only other memory traffic is the job's activation rows, read
// once per job into registers, and the 16 x 8 results per tile.
#include "knj_common.cuh"
#include "knj_q4k.h"
#include "knj_q4k_engine.cuh"

using namespace knj;

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kStages = 4;

struct ProjParams {
  const uint8_t *W0;  // gate (dual) or the single matrix
  const uint8_t *W1;  // up (dual) or null
  const void *X;      // activation rows
  int x_dtype;
  int64_t ldx;
  const int32_t *pair_idx;
  const int32_t *pair_cnt;
  const int32_t *row_map;  // pair -> activation row (null: pair / row_div)
  const int32_t *exp_list;
  const int32_t *n_active;
  float *out0;  // dual: G        single: Y
  float *out1;  // dual: U
  float *out2;  // dual: A = silu(G)*U
  int N, K, row_div, tiles_per_expert;
  int n_experts;  // length of exp_list / pair_cnt
  int ks;         // warps per team = superblocks per row
  int teams;      // teams per CTA
  int64_t idxStride;
  int *status;    // optional: set to 1 when a bounded wait gave up
  long long wait_cycles;  // limit of every wait inside the kernel
  CUtensorMap map0, map1;  // TMA descriptors of W0 / W1: box = one superblock x 8 (dual) or 16 rows
};

struct ProjSmem {
  size_t ring, scratch, red, bars, total;
};
__host__ __device__ inline ProjSmem proj_smem() {
  ProjSmem m;
  m.ring = 0;
  m.scratch = m.ring + (size_t)kWarps * kStages * q4e::kStageBytes;
  m.red = m.scratch + (size_t)kWarps * q4e::kScratchBytes;
  m.bars = m.red + (size_t)2 * kWarps * 32 * sizeof(float4);
  m.total = m.bars + (size_t)kWarps * kStages * 8;
  return m;
}

template <bool DUAL>
__global__ void __launch_bounds__(kThreads, 1) q4k_proj_kernel(const __grid_constant__ ProjParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_jbase[257];  // first job of active expert a (entries past the active ones hold the total)
  __shared__ int s_uexp[256], s_ucnt[256];
  __shared__ int s_fail;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ks = p.ks, team = warp / ks, part = warp - team * ks;
  const ProjSmem lay = proj_smem();
  uint8_t *ring = smem + lay.ring + (size_t)warp * kStages * q4e::kStageBytes;
  uint8_t *scratch = smem + lay.scratch + (size_t)warp * q4e::kScratchBytes;
  float4 *red = reinterpret_cast<float4 *>(smem + lay.red);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + lay.bars) + warp * kStages;

  if (lane == 0)
    for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
  if (threadIdx.x == 0) s_fail = 0;
  mbar_init_fence();
  grid_dep_wait();  // the plan and the activation rows come from earlier launches

  // ---- the job table: jobs per active expert, exclusive prefix (every CTA derives the same table)
  const int n_act = min(p.n_active[0], 256);
  for (int a = threadIdx.x; a < 256; a += kThreads) {
    int c = 0, ex = -1;
    if (a < n_act) {
      ex = p.exp_list[a];
      c = p.pair_cnt[ex];
    }
    s_uexp[a] = ex;
    s_ucnt[a] = c;
    s_jbase[a] = (c + q4e::kMaxTok - 1) / q4e::kMaxTok;
  }
  __syncthreads();
  if (warp == 0) {
    int v[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] = s_jbase[lane * 8 + i]; sum += v[i]; }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    int base = incl - sum;
#pragma unroll
    for (int i = 0; i < 8; ++i) { s_jbase[lane * 8 + i] = base; base += v[i]; }
    if (lane == 31) s_jbase[256] = incl;
  }
  __syncthreads();
  if (team >= p.teams) return;  // warps beyond the last whole team (no CTA-wide barrier follows)

  const int tiles = p.tiles_per_expert;
  const long long U = (long long)s_jbase[256] * tiles;  // < 2^31 (checked by the launcher)
  const long long gteam = (long long)blockIdx.x * p.teams + team, nteams = (long long)gridDim.x * p.teams;
  const int u0 = (int)(U * gteam / nteams), u1 = (int)(U * (gteam + 1) / nteams);
  if (u0 >= u1) return;
  const int rows_per_tile = DUAL ? 8 : 16;
  volatile int *fail = &s_fail;

  // active expert of a job: the last a whose first job is not beyond it
  auto locate = [&](int job) {
    int lo = 0, hi = 255;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_jbase[mid] <= job) lo = mid;
      else hi = mid - 1;
    }
    return lo;
  };

  // ---- producer cursor (lane 0 issues; every lane keeps the same counters)
  int p_job = u0 / tiles, p_tile = u0 - p_job * tiles;
  int p_a = locate(p_job);
  int pu = u0;
  auto issue = [&]() {
    const int stage = (pu - u0) % kStages;
    if (lane == 0) {
      const int row = s_uexp[p_a] * p.N + p_tile * rows_per_tile;
      uint8_t *dst = ring + (size_t)stage * q4e::kStageBytes;
      fence_proxy_async();
      mbar_expect_tx(&bars[stage], (uint32_t)q4e::kStageBytes);
      tma_load_rows(dst, &p.map0, part * (KNJ_Q4K_BYTES / 4), row, &bars[stage]);
      if (DUAL) tma_load_rows(dst + 8 * KNJ_Q4K_BYTES, &p.map1, part * (KNJ_Q4K_BYTES / 4), row, &bars[stage]);
    }
    ++pu;
    if (++p_tile == tiles) {
      p_tile = 0;
      ++p_job;
      while (p_a < 255 && s_jbase[p_a + 1] <= p_job) ++p_a;
    }
  };
  for (int s = 0; s < kStages && pu < u1; ++s) issue();

  // ---- consumer
  q4e::BFrag b;
  q4e::bfrag_clear(b);
  int c_job = u0 / tiles, c_tile = u0 - c_job * tiles;
  int my_pair = -1;
  bool new_job = true, ok = true;
  uint32_t phases = 0;  // bit s: parity the next wait on stage s expects
  int rbuf = 0, rturn = 0;
  for (int u = u0; u < u1; ++u) {
    if (new_job) {
      const int a = locate(c_job);
      const int e = s_uexp[a], cnt = s_ucnt[a];
      const int tok0 = (c_job - s_jbase[a]) * q4e::kMaxTok;
      const int n_tok = min(q4e::kMaxTok, cnt - tok0);
      my_pair = -1;
      int my_row = 0;
      if (lane < n_tok) {
        my_pair = p.pair_idx[(size_t)e * p.idxStride + tok0 + lane];
        my_row = p.row_map ? p.row_map[my_pair] : my_pair / p.row_div;
      }
      // activation rows of the job, four tokens in flight at a time
      for (int j0 = 0; j0 < n_tok; j0 += 4) {
        float v[4][8];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int row = __shfl_sync(0xffffffffu, my_row, min(j0 + jj, n_tok - 1));
          q4e::load8_f32(p.X, p.x_dtype, (int64_t)row * p.ldx + 256 * part + 8 * lane, v[jj]);
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          if (j0 + jj < n_tok) q4e::bfrag_take_token(b, v[jj], j0 + jj, scratch, lane);
      }
      new_job = false;
    }
    const int stage = (u - u0) % kStages;
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok) {
      if (!mbar_wait_for(&bars[stage], (phases >> stage) & 1u, p.wait_cycles, fail)) ok = false;
      phases ^= 1u << stage;
    }
    if (ok) r = q4e::tile_part(ring + (size_t)stage * q4e::kStageBytes, b, lane);
    __syncwarp();  // every lane is done with the stage
    if (ok && pu < u1) issue();

    // ---- the K parts meet (fixed order); the warps of a team take turns as the one that sums and stores
    const int n0 = c_tile * rows_per_tile;
    bool mine = true;
    if (ks > 1) {
      red[(size_t)(rbuf * kWarps + warp) * 32 + lane] = r;
      q4e::team_sync(team, ks * 32);
      mine = part == rturn;
      if (mine) {
        const float4 *src = red + (size_t)(rbuf * kWarps + team * ks) * 32 + lane;
        r = src[0];
        for (int pp = 1; pp < ks; ++pp) {
          const float4 o = src[(size_t)pp * 32];
          r.x += o.x; r.y += o.y; r.z += o.z; r.w += o.w;
        }
      }
      rbuf ^= 1;
      if (++rturn == ks) rturn = 0;
    }
    const int pa = __shfl_sync(0xffffffffu, my_pair, 2 * t), pb = __shfl_sync(0xffffffffu, my_pair, 2 * t + 1);
    if (mine && ok) {
      if (DUAL) {
        const int n = n0 + g;
        if (pa >= 0) {
          const size_t o = (size_t)pa * p.N + n;
          if (p.out0) p.out0[o] = r.x;
          if (p.out1) p.out1[o] = r.z;
          if (p.out2) p.out2[o] = (r.x / (1.0f + expf(-r.x))) * r.z;
        }
        if (pb >= 0) {
          const size_t o = (size_t)pb * p.N + n;
          if (p.out0) p.out0[o] = r.y;
          if (p.out1) p.out1[o] = r.w;
          if (p.out2) p.out2[o] = (r.y / (1.0f + expf(-r.y))) * r.w;
        }
      } else {
        if (pa >= 0) {
          p.out0[(size_t)pa * p.N + n0 + g] = r.x;
          p.out0[(size_t)pa * p.N + n0 + g + 8] = r.z;
        }
        if (pb >= 0) {
          p.out0[(size_t)pb * p.N + n0 + g] = r.y;
          p.out0[(size_t)pb * p.N + n0 + g + 8] = r.w;
        }
      }
    }
    if (++c_tile == tiles) {
      c_tile = 0;
      ++c_job;
      new_job = true;
    }
  }
  if (!ok && lane == 0 && p.status) atomicExch(p.status, 1);
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

long long g_decode_wait_cycles = kMaxWaitCycles;

template <bool DUAL>
int launch_proj(ProjParams p, int n_experts_max, cudaStream_t st) {
  const int nsb = p.K / KNJ_QK_K;
  KNJ_REQUIRE(nsb >= 1 && nsb <= kWarps, "q4k projection: rows of %d weights (at most %d are taken)", p.K, kWarps * KNJ_QK_K);
  KNJ_REQUIRE((long long)n_experts_max * (p.idxStride / q4e::kMaxTok + 1) * p.tiles_per_expert < (1ll << 31),
              "q4k projection: %d experts x %d tiles exceed the work index", n_experts_max, p.tiles_per_expert);
  p.n_experts = n_experts_max;
  p.ks = nsb;
  p.teams = kWarps / nsb;
  p.wait_cycles = g_decode_wait_cycles;
  {
    const uint64_t rows = (uint64_t)n_experts_max * p.N;
    const uint32_t row_bytes = (uint32_t)nsb * KNJ_Q4K_BYTES;
    int rc = make_row_tensor_map(&p.map0, p.W0, rows, row_bytes, KNJ_Q4K_BYTES, DUAL ? 8 : 16);
    if (rc) return rc;
    if (DUAL) {
      rc = make_row_tensor_map(&p.map1, p.W1, rows, row_bytes, KNJ_Q4K_BYTES, 8);
      if (rc) return rc;
    }
  }
  int dev = 0;
  KNJ_CUDA(cudaGetDevice(&dev));
  const size_t smem = proj_smem().total;
  auto kern = q4k_proj_kernel<DUAL>;
  // opt in to the large dynamic shared memory once per device and instantiation
  // (kept out of later launches so they are plain stream work, capturable in a graph)
  static bool opted[64] = {false};
  if (dev >= 0 && dev < 64 && !opted[dev]) {
    KNJ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    opted[dev] = true;
  }
  KNJ_CUDA(launch_chain(kern, dim3((unsigned)sm_count()), dim3(kThreads), smem, st, p));
  return launch_status("q4k_proj_kernel");
}

int check_rows(const void *X, int dtype, int64_t ld, int K, const char *who) {
  KNJ_REQUIRE(dtype >= KNJ_DT_F32 && dtype <= KNJ_DT_F16, "%s: unknown activation dtype %d", who, dtype);
  const int64_t esz = dtype == KNJ_DT_F32 ? 4 : 2;
  KNJ_REQUIRE(aligned16(X) && ld >= K && (ld * esz) % 16 == 0, "%s: activation rows must be 16-byte aligned (ld=%lld)", who,
              (long long)ld);
  return KNJ_OK;
}

}  // namespace

extern "C" {

void knj_decode_wait_limit(long long cycles) { g_decode_wait_cycles = cycles > 0 ? cycles : kMaxWaitCycles; }

int knj_q4k_gateup_launch(const void *X, int x_dtype, int64_t ldx, const uint8_t *Wg, const uint8_t *Wu,
                          const int32_t *pair_idx, const int32_t *pair_cnt, const int32_t *pair_tok,
                          const int32_t *exp_list, const int32_t *n_active, float *G, float *U, float *A, int N, int K,
                          int rowBytes, int64_t idxStride, int n_experts, int top_k, int *status, knj_stream_t s) {
  KNJ_REQUIRE(X && Wg && Wu && pair_idx && pair_cnt && exp_list && n_active, "knj_q4k_gateup: null pointer");
  KNJ_REQUIRE(G || U || A, "knj_q4k_gateup: no output requested");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES,
              "knj_q4k_gateup: rowBytes=%d does not match K=%d", rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % 8 == 0, "knj_q4k_gateup: N=%d must be a multiple of 8", N);
  KNJ_REQUIRE(aligned16(Wg) && aligned16(Wu), "knj_q4k_gateup: weights must be 16-byte aligned");
  KNJ_REQUIRE(n_experts > 0 && n_experts <= 256 && (pair_tok || top_k > 0), "knj_q4k_gateup: bad expert / top_k count");
  int rc = check_rows(X, x_dtype, ldx, K, "knj_q4k_gateup");
  if (rc) return rc;
  ProjParams p{};
  p.W0 = Wg; p.W1 = Wu; p.X = X; p.x_dtype = x_dtype; p.ldx = ldx;
  p.pair_idx = pair_idx; p.pair_cnt = pair_cnt; p.row_map = pair_tok; p.exp_list = exp_list; p.n_active = n_active;
  p.out0 = G; p.out1 = U; p.out2 = A;
  p.N = N; p.K = K; p.row_div = top_k > 0 ? top_k : 1;
  p.tiles_per_expert = N / 8; p.idxStride = idxStride; p.status = status;
  return launch_proj<true>(p, n_experts, as_stream(s));
}

int knj_q4k_proj_launch(const void *A, int a_dtype, int64_t lda, const uint8_t *W, const int32_t *pair_idx,
                        const int32_t *pair_cnt, const int32_t *pair_row, const int32_t *exp_list, const int32_t *n_active,
                        float *Y, int N, int K, int rowBytes, int64_t idxStride, int n_experts, int *status,
                        knj_stream_t s) {
  KNJ_REQUIRE(A && W && pair_idx && pair_cnt && exp_list && n_active && Y, "knj_q4k_proj: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES,
              "knj_q4k_proj: rowBytes=%d does not match K=%d", rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % 16 == 0, "knj_q4k_proj: N=%d must be a multiple of 16", N);
  KNJ_REQUIRE(aligned16(W), "knj_q4k_proj: weights must be 16-byte aligned");
  KNJ_REQUIRE(n_experts > 0 && n_experts <= 256, "knj_q4k_proj: bad expert count");
  int rc = check_rows(A, a_dtype, lda, K, "knj_q4k_proj");
  if (rc) return rc;
  ProjParams p{};
  p.W0 = W; p.W1 = nullptr; p.X = A; p.x_dtype = a_dtype; p.ldx = lda;
  p.pair_idx = pair_idx; p.pair_cnt = pair_cnt; p.row_map = pair_row; p.exp_list = exp_list; p.n_active = n_active;
  p.out0 = Y; p.out1 = nullptr; p.out2 = nullptr;
  p.N = N; p.K = K; p.row_div = 1;
  p.tiles_per_expert = N / 16; p.idxStride = idxStride; p.status = status;
  return launch_proj<false>(p, n_experts, as_stream(s));
}

size_t knj_q4k_matmul_workspace_bytes(int m, int n_in) {
  if (m <= 0 || n_in <= 0) return 0;
  // identity pair list + counts
  return (((size_t)m * 4 + 255) & ~(size_t)255) + 256;
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
  int32_t *pair_idx = reinterpret_cast<int32_t *>(ws);
  ws += ((size_t)m * 4 + 255) & ~(size_t)255;
  int32_t *small = reinterpret_cast<int32_t *>(ws);  // [0] cnt, [1] exp_list, [2..3] n_active
  iota_plan_kernel<<<(m + 255) / 256, 256, 0, as_stream(s)>>>(pair_idx, small + 0, small + 1, small + 2, m);
  int rc = launch_status("iota_plan_kernel");
  if (rc) return rc;
  return knj_q4k_proj_launch(x, x_dtype, ldx, W, pair_idx, small + 0, nullptr, small + 1, small + 2, y, n_out, n_in,
                             n_in / 256 * KNJ_Q4K_BYTES, m, 1, nullptr, s);
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
