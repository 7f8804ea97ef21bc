// knj_q4k_mma.cu -- decode-class expert projections as stand-alone launches:
// gate+up+SiLU*up (tools/bench/q4k_moe_ffn.hip:164-241 knj_q4k_gateup fused with
// tools/bench/q4k_stream_ffn.hip:1021-1031), the single-matrix projection
// (tools/bench/q4k_stream_ffn.hip:834-882 knj_q4k_proj) and Model::matmul
// (src/model/model.cpp:326-380), all on the tile engine of knj_q4k_engine.cuh.
//
// One persistent CTA per SM, 16 independent warps. The work of a launch is the
// flat list (job, tile): a JOB is one active expert with up to 8 of its tokens (an
// expert with more tokens yields several jobs; its weights then come from L2 after
// the first), a tile is 16 weight rows. Every CTA takes an equal contiguous run of
// that list, one job at a time: the CTA converts the job's activation rows into a
// shared-memory panel once, then warp w takes every 16th tile of the run, walks its
// superblocks through its own ring of TMA boxes (filled `stages` boxes ahead, across
// tile boundaries) and stores the 16 x 8 results itself. No partial sums cross warps
// and nothing but weights and the panel is read in the inner loop.
#include "knj_common.cuh"
#include "knj_q4k.h"
#include "knj_q4k_engine.cuh"

using namespace knj;

namespace {

constexpr int kThreads = q4e::kWarps * 32;

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
  int K, row_div;
  int n_experts;  // length of exp_list / pair_cnt
  q4e::PhaseShape shape;
  int64_t idxStride;
  int *status;    // optional: set to 1 when a bounded wait gave up
  long long wait_cycles;   // limit of every wait inside the kernel
  CUtensorMap map0, map1;  // TMA descriptors of W0 / W1: box = sbs superblocks x 8 (dual) or 16 rows
};

struct ProjSmem {
  size_t ring, panels, bars, red, total;
};
__host__ __device__ inline ProjSmem proj_smem(int nsb, int sbs, int stages) {
  ProjSmem m;
  m.ring = 0;
  m.panels = m.ring + q4e::phase_ring_bytes(sbs, stages);
  m.bars = m.panels + q4e::phase_panel_bytes(nsb);
  m.red = m.bars + (size_t)q4e::kWarps * q4e::kMaxStages * 8;
  m.total = m.red + (size_t)q4e::kWarps * 32 * sizeof(float4);
  return m;
}

#ifdef KNJ_TRACE
// Measurement build only: experiment modes (1: no arithmetic; 2: no weight copies; 3: no activation panels).
__device__ int g_trace_mode = 0;
#endif

template <bool DUAL>
__global__ void __launch_bounds__(kThreads, 1) q4k_proj_kernel(const __grid_constant__ ProjParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_jbase[257];
  __shared__ int s_uexp[256], s_ucnt[256];
  __shared__ float s_inv[q4e::kJobTok * 16];
  __shared__ int s_pair[q4e::kJobTok];
  __shared__ int s_fail;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const ProjSmem lay = proj_smem(p.shape.nsb, p.shape.sbs, p.shape.stages);
  q4e::PhaseSmem sm;
  sm.ring = smem + lay.ring;
  sm.panels = smem + lay.panels;
  sm.bars = reinterpret_cast<uint64_t *>(smem + lay.bars);
  sm.red = reinterpret_cast<float4 *>(smem + lay.red);
  sm.inv = s_inv;
  sm.pair = s_pair;
  sm.fail = &s_fail;
  if (lane == 0)
    for (int s = 0; s < q4e::kMaxStages; ++s) mbar_init(&sm.bars[warp * q4e::kMaxStages + s], 1);
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
    s_jbase[a] = (c + q4e::kJobTok - 1) / q4e::kJobTok;
  }
  __syncthreads();
  if (warp == 0) q4e::job_prefix(s_jbase, lane);
  __syncthreads();

  const long long U = (long long)s_jbase[256] * p.shape.tiles;  // < 2^31 (checked by the launcher)
  const int u0 = (int)(U * blockIdx.x / gridDim.x), u1 = (int)(U * (blockIdx.x + 1) / gridDim.x);
  q4e::JobTable jt{s_jbase, s_uexp};
  unsigned parity = 0;
  bool ok = true;
  int tmode = 0;
#ifdef KNJ_TRACE
  tmode = g_trace_mode;
#endif
  q4e::run_phase<DUAL>(
      p.shape, sm, jt, u0, u1, q4e::choose_ksplit(U, p.shape.nsb / p.shape.sbs, gridDim.x), &p.map0, &p.map1, p.out0, p.out1, p.out2, p.wait_cycles, parity, ok,
      [&](int job, int a, int tk, int &pair, int &row) {
        const int tok = (job - s_jbase[a]) * q4e::kJobTok + tk;
        if (tok >= s_ucnt[a]) return false;
        pair = p.pair_idx[(size_t)s_uexp[a] * p.idxStride + tok];
        row = p.row_map ? p.row_map[pair] : pair / p.row_div;
        return true;
      },
      [&](int row, int sb, int ln, float (&v)[8]) { q4e::load8_f32(p.X, p.x_dtype, (int64_t)row * p.ldx + 256 * sb + 8 * ln, v); },
      tmode);
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
  KNJ_REQUIRE(nsb >= 1 && nsb <= 16, "q4k projection: rows of %d weights (at most 4096 are taken)", p.K);
  KNJ_REQUIRE((long long)n_experts_max * (p.idxStride / q4e::kJobTok + 1) * p.shape.tiles < (1ll << 31),
              "q4k projection: %d experts x %d tiles exceed the work index", n_experts_max, p.shape.tiles);
  p.n_experts = n_experts_max;
  p.shape.nsb = nsb;
  p.shape.sbs = (nsb % 2 == 0) ? 2 : 1;
  p.wait_cycles = g_decode_wait_cycles;
  {
    const uint64_t rows = (uint64_t)n_experts_max * p.shape.N;
    const uint32_t box = (uint32_t)p.shape.sbs * KNJ_Q4K_BYTES;
    int rc = make_row_tensor_map(&p.map0, p.W0, rows, (uint32_t)nsb * KNJ_Q4K_BYTES, box, DUAL ? 8 : 16);
    if (rc) return rc;
    if (DUAL) {
      rc = make_row_tensor_map(&p.map1, p.W1, rows, (uint32_t)nsb * KNJ_Q4K_BYTES, box, 8);
      if (rc) return rc;
    }
  }
  int dev = 0;
  KNJ_CUDA(cudaGetDevice(&dev));
  int smem_max = 0;
  KNJ_CUDA(cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  const size_t reserve = 6 * 1024;  // the kernel's static shared memory
  p.shape.stages = p.shape.sbs == 2 ? 2 : q4e::kMaxStages;  // four superblocks in flight per warp either way
  while (p.shape.stages > 2 && proj_smem(nsb, p.shape.sbs, p.shape.stages).total + reserve > (size_t)smem_max) --p.shape.stages;
  const size_t smem = proj_smem(nsb, p.shape.sbs, p.shape.stages).total;
  KNJ_REQUIRE(smem + reserve <= (size_t)smem_max, "q4k projection: rows of %d weights do not fit the shared memory", p.K);
  auto kern = q4k_proj_kernel<DUAL>;
  // opt in to the large dynamic shared memory once per device and instantiation
  // (kept out of later launches so they are plain stream work, capturable in a graph)
  static size_t opted[64] = {0};
  if (dev >= 0 && dev < 64 && opted[dev] < smem) {
    KNJ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    opted[dev] = smem;
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

namespace knj {
long long decode_wait_cycles() { return g_decode_wait_cycles; }
}  // namespace knj

extern "C" {

#ifdef KNJ_TRACE
int knj_trace_proj(long long *, int mode) {  // measurement build only
  KNJ_CUDA(cudaMemcpyToSymbol(g_trace_mode, &mode, sizeof(mode)));
  return KNJ_OK;
}
int knj_trace_feed(int) { return 0; }
#endif

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
  p.shape.N = N; p.K = K; p.row_div = top_k > 0 ? top_k : 1;
  p.shape.tiles = N / 8; p.idxStride = idxStride; p.status = status;
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
  p.shape.N = N; p.K = K; p.row_div = 1;
  p.shape.tiles = N / 16; p.idxStride = idxStride; p.status = status;
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
constexpr size_t kNoAllocScratchBytes = (size_t)64 << 10;  // 64 KiB: the pair list of up to 16,256 activation rows
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
