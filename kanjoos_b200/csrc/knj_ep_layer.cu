// knj_ep_layer.cu -- the expert-parallel MoE-FFN layer of one rank as a C-ABI
// object: experts split contiguously over the ranks (owner(e) = e / (E / world)),
// tokens data-parallel, one process per GPU, every rank's exchange buffers mapped
// into every process (NVLink peer mappings supplied by the host, e.g. CUDA IPC or
// symmetric memory). The reference keeps every expert on one device and has no
// counterpart (multi-GPU is a declared non-goal there, README.md:104-107); the
// per-rank arithmetic is the single-GPU layer's (src/model/model.cpp:399-510).
//
// One step on one rank:
//   side stream : the rank's token rows, converted to fp16, are STORED into every
//                 rank's gathered-rows buffer (peer stores: the data crosses NVLink
//                 once per destination while the router below runs)
//   main stream : router logits + top-k straight into the rank's slice of its own
//                 gathered routing tables, then the slice is stored to the peers
//   flag barrier: every rank has written a new epoch into every peer's flag array
//                 and seen all of them (plain peer stores and loads, bounded spin)
//   plan over the global pair list restricted to the rank's experts, the two
//   grouped tensor-core GEMMs over its experts (rows are read through pair / top_k,
//   no per-pair copies), the rank's weighted partial sum of every token stored
//   into the token owner's `parts[rank]` slot, flag barrier, and the sum over the
//   contributing ranks in ascending rank order (+ residual).
// No collective library call is on this path; NCCL or any other transport is only
// what the host used to exchange the buffer addresses at set-up. No multicast and
// no bulk copies: peer memory is touched by plain loads and stores of this file's
// kernels only, the GEMMs read local memory.
#include "knj_common.cuh"
#include "knj_q4k.h"
#include "knj_q4k_engine.cuh"

#include <vector>

using namespace knj;

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier over the ranks, on the stream: thread j tells rank j that this rank has reached epoch e (a store into
// slot `rank` of j's flag words) and waits until rank j has told this rank the same (slot j of the own words).
// Everything this rank stored into peer memory before the launch is visible to a peer that leaves its barrier.
// A wait that runs out of time raises *status and the kernel returns; nothing spins without a limit.
__global__ void ep_barrier_kernel(uint32_t *const *flags, int slot, int world, int rank, uint32_t *epoch, long long limit, int *status) {
  const int j = threadIdx.x;
  const uint32_t e = *epoch + 1u;
  __threadfence_system();
  if (j < world) {
    st_release_sys(flags[j] + slot + rank, e);
    const uint32_t *mine = flags[rank] + slot + j;
    const long long t0 = clock64();
    unsigned polls = 0;
    while ((int32_t)(ld_acquire_sys(mine) - e) < 0) {
      if ((++polls & 255u) == 0u && clock64() - t0 > limit) {
        atomicExch(status, 1);
        break;
      }
    }
  }
  __syncthreads();
  if (j == 0) *epoch = e;
}

// The two halves of that barrier as launches of their own, so that they can sit on different streams: the arrival
// follows the kernel whose peer stores it announces (the copy stream), the wait precedes the kernel that reads
// what the peers stored (the compute stream). e is the step number, the same on every rank.
__global__ void ep_arrive_kernel(uint32_t *const *flags, int slot, int world, int rank, uint32_t e) {
  __threadfence_system();
  if ((int)threadIdx.x < world) st_release_sys(flags[threadIdx.x] + slot + rank, e);
}
__global__ void ep_wait_kernel(const uint32_t *mine, int world, uint32_t e, long long limit, int *status) {
  if ((int)threadIdx.x < world) {
    const long long t0 = clock64();
    unsigned polls = 0;
    while ((int32_t)(ld_acquire_sys(mine + threadIdx.x) - e) < 0) {
      if ((++polls & 255u) == 0u && clock64() - t0 > limit) {
        atomicExch(status, 1);
        break;
      }
    }
  }
  __threadfence_system();
}

// The rank's fp16 rows (already in its own slot of the gathered-rows buffer) to the same place in every peer's
// buffer, as 16-byte stores. The grid is cut into world-1 phases of `cpp` CTAs; phase i stores to rank
// (rank + 1 + i) % world, and CTAs start in block order, so at any moment every rank is writing to a different peer
// (all ranks storing to the same peer at once shares that peer's ingress: measured 2x slower).
__global__ void __launch_bounds__(256) ep_push_rows_kernel(const uint4 *__restrict__ src, __half *const *__restrict__ dst, int64_t off16,
                                                           int64_t n16, int world, int rank, int cpp) {
  const int phase = blockIdx.x / cpp, b = blockIdx.x - phase * cpp;
  int d = rank + 1 + phase;
  if (d >= world) d -= world;
  uint4 *out = reinterpret_cast<uint4 *>(dst[d]) + off16;
  const int64_t stride = (int64_t)cpp * 256;
  for (int64_t i = (int64_t)b * 256 + threadIdx.x; i < n16; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * stride < n16) v[u] = __ldg(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * stride < n16) out[i + u * stride] = v[u];
  }
}

// The rank's routing tables (local order, [T_loc*k]) into every rank's gathered tables: the slice of chunk c goes
// to element c*chunk_stride + rank_off (16 bytes per thread).
__global__ void __launch_bounds__(256) ep_push_tables_kernel(const int32_t *__restrict__ pe_loc, const float *__restrict__ pw_loc,
                                                             int32_t *const *__restrict__ pe, float *const *__restrict__ pw, int world,
                                                             int64_t n4, int64_t n4_chunk, int64_t chunk_stride, int64_t rank_off) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 a = reinterpret_cast<const uint4 *>(pe_loc)[i], b = reinterpret_cast<const uint4 *>(pw_loc)[i];
    const int64_t c = i / n4_chunk, at = c * chunk_stride + rank_off + 4 * (i - c * n4_chunk);
    for (int d = 0; d < world; ++d) {
      *reinterpret_cast<uint4 *>(pe[d] + at) = a;
      *reinterpret_cast<uint4 *>(pw[d] + at) = b;
    }
  }
}

// expert ids of the global pair list relative to this rank's first expert; foreign experts become -1
__global__ void __launch_bounds__(256) ep_local_ids_kernel(const int32_t *__restrict__ pe, int lo, int e_loc, int n, int32_t *__restrict__ out) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int e = pe[i] - lo;
    out[i] = (e >= 0 && e < e_loc) ? e : -1;
  }
}

inline size_t up256(size_t n) { return (n + 255) & ~(size_t)255; }

}  // namespace

struct knj_ep_ctx {
  knj_ep_desc d{};
  int C = 1;                      // chunks of a step
  int Tc_loc = 0, Tc = 0, Pc = 0, e_loc = 0;  // per chunk: local tokens, tokens of all ranks, pairs of all ranks
  char *block = nullptr;          // one device allocation, carved below
  // device copies of the pointer tables
  __half **xall_ptrs = nullptr;
  int32_t **pe_ptrs = nullptr;
  float **pw_ptrs = nullptr;
  float **parts_ptrs = nullptr;
  uint32_t **flag_ptrs = nullptr;
  // this rank's own buffers (entries `rank` of the tables)
  __half *x_all = nullptr;
  int32_t *pe_all = nullptr;
  float *pw_all = nullptr;
  float *parts = nullptr;
  uint32_t *flags = nullptr;
  // local scratch
  float *logits = nullptr, *pw_loc = nullptr, *Y[2] = {nullptr, nullptr};
  int32_t *pe_loc = nullptr, *local_ids = nullptr, *pair_idx = nullptr, *pair_cnt = nullptr, *exp_list = nullptr, *n_active = nullptr;
  void *perm_scratch = nullptr, *ah = nullptr;
  size_t perm_bytes = 0;
  uint32_t *epoch = nullptr;
  int *status = nullptr;  // [0] rank waits, [1] GEMMs
  long long wait_cycles = kMaxWaitCycles;
  uint32_t step = 0;      // steps launched so far: the epoch the flag words of a step carry
  int transport = KNJ_EP_SM_PARTIALS | KNJ_EP_F16_PARTIALS;
  std::vector<__half *> h_xall;  // host copies of two pointer tables, for the block copies
  std::vector<float *> h_parts;
  float *stage[2] = {nullptr, nullptr};  // partial rows of other ranks' tokens before their block copies, by chunk parity
  cudaStream_t side = nullptr, side2 = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_router = nullptr, ev_side = nullptr, ev_a = nullptr, ev_b = nullptr;
  cudaEvent_t ev_down[KNJ_EP_MAX_CHUNKS] = {}, ev_sent[KNJ_EP_MAX_CHUNKS] = {};
#ifdef KNJ_TRACE
  cudaEvent_t stamp[12] = {};
#endif
};

#ifdef KNJ_TRACE
#define KNJ_EP_STAMP(i)                                                        \
  do {                                                                         \
    if (!c->stamp[i]) cudaEventCreate(&c->stamp[i]);                           \
    cudaEventRecord(c->stamp[i], st);                                          \
  } while (0)
#else
#define KNJ_EP_STAMP(i) ((void)0)
#endif

// flag words of a rank: [0, C*world) rows and tables of chunk c have been stored; [C*world, 2*C*world) partial
// sums of chunk c have been stored; kBarrierSlot.. the stand-alone barrier
static constexpr int kBarrierSlot = KNJ_EP_FLAG_WORDS - 64;

extern "C" {

int knj_ep_create(const knj_ep_desc *desc, knj_ep_ctx **out) {
  KNJ_REQUIRE(desc && out, "knj_ep_create: null argument");
  *out = nullptr;
  const knj_ep_desc &d = *desc;
  const int C = d.n_chunks <= 0 ? 1 : d.n_chunks;
  KNJ_REQUIRE(d.world >= 1 && d.world <= 64 && d.rank >= 0 && d.rank < d.world, "knj_ep_create: rank %d of %d", d.rank, d.world);
  KNJ_REQUIRE(d.n_experts >= d.world && d.n_experts % d.world == 0 && d.n_experts / d.world <= 256,
              "knj_ep_create: %d experts do not split over %d ranks", d.n_experts, d.world);
  KNJ_REQUIRE(d.n_tokens_local >= 1 && d.hidden > 0 && d.ffn > 0 && d.hidden % 256 == 0 && d.ffn % 256 == 0,
              "knj_ep_create: bad token count / hidden / ffn");
  KNJ_REQUIRE(C <= KNJ_EP_MAX_CHUNKS && d.n_tokens_local % C == 0 && 2 * C * d.world <= kBarrierSlot,
              "knj_ep_create: %d local tokens do not split into %d chunks", d.n_tokens_local, C);
  KNJ_REQUIRE(d.top_k >= 1 && d.top_k <= 8 && ((int64_t)(d.n_tokens_local / C) * d.top_k) % 4 == 0,
              "knj_ep_create: top_k out of range or a chunk's local pairs not a multiple of 4");
  KNJ_REQUIRE(d.xall_ptrs && d.pe_ptrs && d.pw_ptrs && d.parts_ptrs && d.flag_ptrs, "knj_ep_create: null pointer table");
  for (int r = 0; r < d.world; ++r)
    KNJ_REQUIRE(d.xall_ptrs[r] && d.pe_ptrs[r] && d.pw_ptrs[r] && d.parts_ptrs[r] && d.flag_ptrs[r] && aligned16(d.xall_ptrs[r]) &&
                    aligned16(d.pe_ptrs[r]) && aligned16(d.pw_ptrs[r]) && aligned16(d.parts_ptrs[r]),
                "knj_ep_create: rank %d's buffers are missing or not 16-byte aligned", r);
  knj_ep_ctx *c = new knj_ep_ctx();
  c->d = d;
  c->C = C;
  c->Tc_loc = d.n_tokens_local / C;
  c->Tc = c->Tc_loc * d.world;
  c->Pc = c->Tc * d.top_k;
  c->e_loc = d.n_experts / d.world;
  const size_t Tc = c->Tc, Pc = c->Pc, H = d.hidden, F = d.ffn, W = d.world, Pl = (size_t)d.n_tokens_local * d.top_k;
  c->perm_bytes = knj_moe_permute_scratch_bytes(c->Pc, c->e_loc);
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t at = off; off += up256(bytes); return at; };
  const size_t o_tab = take(5 * W * sizeof(void *));
  const size_t o_logits = take((size_t)d.n_tokens_local * d.n_experts * 4);
  const size_t o_pe = take(Pl * 4), o_pw = take(Pl * 4);
  const size_t o_ids = take(Pc * 4);
  const size_t o_pidx = take((size_t)c->e_loc * Tc * 4);
  const size_t o_small = take((size_t)(2 * c->e_loc + 16) * 4);
  const size_t o_perm = take(c->perm_bytes);
  const size_t o_ah = take(Pc * F * 2);
  const size_t o_y0 = take(Pc * H * 4);
  const size_t o_y1 = C > 1 ? take(Pc * H * 4) : o_y0;
  const size_t o_st0 = take(Tc * H * 4);
  const size_t o_st1 = C > 1 ? take(Tc * H * 4) : o_st0;
  const size_t o_words = take(64);
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&c->block), off);
  if (e == cudaSuccess) e = cudaMemset(c->block + o_words, 0, 64);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->side2, cudaStreamNonBlocking);
  cudaEvent_t *evs[5] = {&c->ev_fork, &c->ev_router, &c->ev_side, &c->ev_a, &c->ev_b};
  for (int i = 0; i < 5 && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(evs[i], cudaEventDisableTiming);
  for (int i = 0; i < C && e == cudaSuccess; ++i) {
    e = cudaEventCreateWithFlags(&c->ev_down[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_sent[i], cudaEventDisableTiming);
  }
  void **tab = c->block ? reinterpret_cast<void **>(c->block + o_tab) : nullptr;
  const void *const *src[5] = {d.xall_ptrs, reinterpret_cast<const void *const *>(d.pe_ptrs), reinterpret_cast<const void *const *>(d.pw_ptrs),
                               reinterpret_cast<const void *const *>(d.parts_ptrs), reinterpret_cast<const void *const *>(d.flag_ptrs)};
  for (int i = 0; i < 5 && e == cudaSuccess; ++i) e = cudaMemcpy(tab + i * W, src[i], W * sizeof(void *), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    knj_ep_destroy(c);
    cudaGetLastError();
    set_error("knj_ep_create: device set-up failed (%s)", cudaGetErrorString(e));
    return KNJ_E_RUNTIME;
  }
  c->xall_ptrs = reinterpret_cast<__half **>(tab);
  c->pe_ptrs = reinterpret_cast<int32_t **>(tab + W);
  c->pw_ptrs = reinterpret_cast<float **>(tab + 2 * W);
  c->parts_ptrs = reinterpret_cast<float **>(tab + 3 * W);
  c->flag_ptrs = reinterpret_cast<uint32_t **>(tab + 4 * W);
  c->x_all = static_cast<__half *>(d.xall_ptrs[d.rank]);
  c->pe_all = d.pe_ptrs[d.rank];
  c->pw_all = d.pw_ptrs[d.rank];
  c->parts = d.parts_ptrs[d.rank];
  c->flags = d.flag_ptrs[d.rank];
  c->logits = reinterpret_cast<float *>(c->block + o_logits);
  c->pe_loc = reinterpret_cast<int32_t *>(c->block + o_pe);
  c->pw_loc = reinterpret_cast<float *>(c->block + o_pw);
  c->local_ids = reinterpret_cast<int32_t *>(c->block + o_ids);
  c->pair_idx = reinterpret_cast<int32_t *>(c->block + o_pidx);
  c->pair_cnt = reinterpret_cast<int32_t *>(c->block + o_small);
  c->exp_list = c->pair_cnt + c->e_loc;
  c->n_active = c->exp_list + c->e_loc;
  c->perm_scratch = c->block + o_perm;
  c->ah = c->block + o_ah;
  c->Y[0] = reinterpret_cast<float *>(c->block + o_y0);
  c->Y[1] = reinterpret_cast<float *>(c->block + o_y1);
  c->stage[0] = reinterpret_cast<float *>(c->block + o_st0);
  c->stage[1] = reinterpret_cast<float *>(c->block + o_st1);
  for (int r = 0; r < d.world; ++r) {
    c->h_xall.push_back(static_cast<__half *>(d.xall_ptrs[r]));
    c->h_parts.push_back(d.parts_ptrs[r]);
  }
  c->epoch = reinterpret_cast<uint32_t *>(c->block + o_words);
  c->status = reinterpret_cast<int *>(c->block + o_words + 16);
  *out = c;
  return KNJ_OK;
}

int knj_ep_set_wait(knj_ep_ctx *c, long long wait_cycles) {
  KNJ_REQUIRE(c, "knj_ep_set_wait: null context");
  c->wait_cycles = wait_cycles > 0 ? wait_cycles : kMaxWaitCycles;
  return KNJ_OK;
}

int knj_ep_set_transport(knj_ep_ctx *c, int transport) {
  KNJ_REQUIRE(c && transport >= 0 && transport <= (KNJ_EP_SM_ROWS | KNJ_EP_SM_PARTIALS | KNJ_EP_F16_PARTIALS), "knj_ep_set_transport: unknown transport");
  c->transport = transport;
  return KNJ_OK;
}

int knj_ep_barrier_launch(knj_ep_ctx *c, knj_stream_t s) {
  KNJ_REQUIRE(c && c->block, "knj_ep_barrier: null context");
  ep_barrier_kernel<<<1, 64, 0, as_stream(s)>>>(c->flag_ptrs, kBarrierSlot, c->d.world, c->d.rank, c->epoch, c->wait_cycles, c->status);
  return launch_status("ep_barrier_kernel");
}

int knj_ep_forward_launch(knj_ep_ctx *c, const void *x, int x_dtype, int64_t ldx, const uint16_t *w_router,
                          const float *router_bias, const uint8_t *w_gate, const uint8_t *w_up, const uint8_t *w_down,
                          int residual, void *out, int out_dtype, knj_stream_t s) {
  KNJ_REQUIRE(c && c->block && x && w_router && w_gate && w_up && w_down && out, "knj_ep_forward: null pointer");
  KNJ_REQUIRE(x_dtype == KNJ_DT_F32 || x_dtype == KNJ_DT_BF16 || x_dtype == KNJ_DT_F16, "knj_ep_forward: unknown x dtype");
  KNJ_REQUIRE(out_dtype == KNJ_DT_F32 || out_dtype == KNJ_DT_BF16, "knj_ep_forward: out must be f32 or bf16");
  const knj_ep_desc &d = c->d;
  const int T_loc = d.n_tokens_local, H = d.hidden, F = d.ffn, k = d.top_k, W = d.world, rank = d.rank, C = c->C;
  const int Tc_loc = c->Tc_loc, Tc = c->Tc, Pc = c->Pc;
  KNJ_REQUIRE(ldx >= H && ldx % 8 == 0 && aligned16(x) && (!residual || ldx == H), "knj_ep_forward: rows of x must be 16-byte aligned (dense with residual)");
  cudaStream_t st = as_stream(s), side = c->side;
  const size_t x_el = x_dtype == KNJ_DT_F32 ? 4 : 2, o_el = out_dtype == KNJ_DT_F32 ? 4 : 2;
  const uint32_t epoch = ++c->step;
  int rc;
  KNJ_EP_STAMP(0);
  KNJ_CUDA(cudaMemsetAsync(c->status, 0, 2 * sizeof(int), st));
  // ---- main stream: the first chunk's rows as fp16 (ahead of the router, so that their copies run beside it), then
  //      the router over all local tokens (tables in local order)
  const bool ce = !(c->transport & KNJ_EP_SM_ROWS), ce_parts = !(c->transport & KNJ_EP_SM_PARTIALS);
  // partial rows as fp16 under a per-row scale: only in the form the combining kernel stores itself
  const bool f16p = (c->transport & KNJ_EP_F16_PARTIALS) && !ce_parts && H <= 2048;
  rc = knj_to_f16_launch(x, x_dtype, ldx, Tc_loc, H, c->x_all + (int64_t)rank * Tc_loc * H, s);
  if (rc) return rc;
  KNJ_CUDA(cudaEventRecord(c->ev_fork, st));
  KNJ_CUDA(cudaStreamWaitEvent(side, c->ev_fork, 0));
  KNJ_CUDA(cudaStreamWaitEvent(c->side2, c->ev_fork, 0));
  rc = knj_router_topk_launch(x, x_dtype, ldx, w_router, router_bias, T_loc, H, d.n_experts, k, c->logits, c->pe_loc, c->pw_loc, s);
  if (rc) return rc;
  KNJ_CUDA(cudaEventRecord(c->ev_router, st));
  KNJ_EP_STAMP(1);
  // ---- copy streams: chunk by chunk the rows to every rank, the tables once, an arrival per chunk
  cudaStream_t side2 = c->side2;
  // block copies go to the nearest higher rank first (at any moment a rank receives from one sender), alternating
  // over the two copy streams so that one copy's start-up hides behind the other's transfer; joined on `side`
  for (int ch = 0; ch < C; ++ch) {
    const int64_t off = ((int64_t)ch * Tc + (int64_t)rank * Tc_loc) * H;
    const void *xc = static_cast<const char *>(x) + (size_t)ch * Tc_loc * ldx * x_el;
    if (ch > 0) {
      rc = knj_to_f16_launch(xc, x_dtype, ldx, Tc_loc, H, c->x_all + off, side);
      if (rc) return rc;
    }
    if (!ce && W > 1) {  // staggered stores of the library's own kernel
      const int64_t n16 = (int64_t)Tc_loc * H / 8;
      int cpp = (int)((n16 + 1023) / 1024);
      if (cpp > 2 * sm_count()) cpp = 2 * sm_count();
      ep_push_rows_kernel<<<(unsigned)(cpp * (W - 1)), 256, 0, side>>>(reinterpret_cast<const uint4 *>(c->x_all + off), c->xall_ptrs, off / 8, n16, W,
                                                                      rank, cpp);
      rc = launch_status("ep_push_rows_kernel");
      if (rc) return rc;
    }
    if (ce && W > 1) {  // the block copies start before the tables below wait for the router
      KNJ_CUDA(cudaEventRecord(c->ev_a, side));
      KNJ_CUDA(cudaStreamWaitEvent(side2, c->ev_a, 0));
      for (int i = 1; i < W; ++i) {
        const int dr = (rank + i) % W;
        KNJ_CUDA(cudaMemcpyAsync(c->h_xall[dr] + off, c->x_all + off, (size_t)Tc_loc * H * 2, cudaMemcpyDeviceToDevice, (i & 1) ? side2 : side));
      }
      KNJ_CUDA(cudaEventRecord(c->ev_b, side2));
    }
    if (ch == 0) {
      KNJ_CUDA(cudaStreamWaitEvent(side, c->ev_router, 0));
      const int64_t n4 = (int64_t)T_loc * k / 4, n4c = (int64_t)Tc_loc * k / 4;
      ep_push_tables_kernel<<<(unsigned)((n4 + 255) / 256 < 592 ? (n4 + 255) / 256 : 592), 256, 0, side>>>(
          c->pe_loc, c->pw_loc, c->pe_ptrs, c->pw_ptrs, W, n4, n4c, (int64_t)Pc, (int64_t)rank * Tc_loc * k);
      rc = launch_status("ep_push_tables_kernel");
      if (rc) return rc;
    }
    if (ce && W > 1) KNJ_CUDA(cudaStreamWaitEvent(side, c->ev_b, 0));
    ep_arrive_kernel<<<1, 64, 0, side>>>(c->flag_ptrs, ch * W, W, rank, epoch);
    rc = launch_status("ep_arrive_kernel");
    if (rc) return rc;
  }
  // ---- main stream: per chunk the rank's experts over the chunk's tokens of all ranks; the partial sums leave
  //      on the copy stream while the next chunk's GEMMs run
  const int lo = rank * c->e_loc;
  auto reduce_chunk = [&](int ch) -> int {
    ep_wait_kernel<<<1, 64, 0, st>>>(c->flags + (C + ch) * W, W, epoch, c->wait_cycles, c->status);
    int r2 = launch_status("ep_wait_kernel");
    if (r2) return r2;
    const void *res = residual ? static_cast<const char *>(x) + (size_t)ch * Tc_loc * ldx * x_el : nullptr;
    void *o = static_cast<char *>(out) + (size_t)ch * Tc_loc * H * o_el;
    if (f16p)
      return ep_reduce_sel_f16(c->parts + (size_t)ch * Tc * H, W, Tc_loc, H, c->pe_loc + (size_t)ch * Tc_loc * k, k, c->e_loc, res, x_dtype, o,
                               out_dtype, st);
    return knj_ep_reduce_sel_launch(c->parts + (size_t)ch * Tc * H, W, Tc_loc, H, c->pe_loc + (size_t)ch * Tc_loc * k, k, c->e_loc, res,
                                    x_dtype, o, out_dtype, s);
  };
  for (int ch = 0; ch < C; ++ch) {
    const __half *xa = c->x_all + (size_t)ch * Tc * H;
    const int32_t *pe = c->pe_all + (size_t)ch * Pc;
    const float *pw = c->pw_all + (size_t)ch * Pc;
    float *Y = c->Y[ch & 1];
    if (ch == 0) KNJ_EP_STAMP(2);
    ep_wait_kernel<<<1, 64, 0, st>>>(c->flags + ch * W, W, epoch, c->wait_cycles, c->status);
    rc = launch_status("ep_wait_kernel");
    if (rc) return rc;
    if (ch == 0) KNJ_EP_STAMP(3);
    ep_local_ids_kernel<<<(unsigned)((Pc + 255) / 256 < 1184 ? (Pc + 255) / 256 : 1184), 256, 0, st>>>(pe, lo, c->e_loc, Pc, c->local_ids);
    rc = launch_status("ep_local_ids_kernel");
    if (rc) return rc;
    rc = knj_moe_permute_ws_launch(c->local_ids, Pc, c->e_loc, Tc, c->pair_idx, c->pair_cnt, c->exp_list, c->n_active, c->perm_scratch,
                                   c->perm_bytes, s);
    if (rc) return rc;
    if (ch == 0) KNJ_EP_STAMP(4);
    rc = knj_q4k_gateup_tc_launch(xa, w_gate, w_up, c->pair_idx, c->pair_cnt, nullptr, c->ah, F, H, H / 256 * KNJ_Q4K_BYTES, Tc, c->e_loc, k,
                                  Pc, c->status + 1, s);
    if (rc) return rc;
    if (ch == 0) KNJ_EP_STAMP(5);
    if (ch >= 2) KNJ_CUDA(cudaStreamWaitEvent(st, c->ev_sent[ch - 2], 0));  // the rows of Y[ch & 1] / stage[ch & 1] have left
    rc = knj_q4k_down_tc_launch(c->ah, w_down, c->pair_idx, c->pair_cnt, nullptr, Y, H, F, F / 256 * KNJ_Q4K_BYTES, Tc, c->e_loc, Pc,
                                c->status + 1, s);
    if (rc) return rc;
    if (ch == 0) KNJ_EP_STAMP(6);
    // weighted partial sums of the chunk to the token owners, then the arrival
    if (ce_parts) {
      // the sums on this stream: own tokens' rows into the own array, the others' staged by owner; block copies follow
      float *stg = c->stage[ch & 1];
      rc = ep_combine_partial_peer_at(Y, pe, pw, Tc, H, k, lo, lo + c->e_loc, c->parts_ptrs, (int64_t)ch * Tc * H, stg, rank, Tc_loc, st);
      if (rc) return rc;
      KNJ_CUDA(cudaEventRecord(c->ev_down[ch], st));
      KNJ_CUDA(cudaStreamWaitEvent(side, c->ev_down[ch], 0));
      KNJ_CUDA(cudaStreamWaitEvent(side2, c->ev_down[ch], 0));
      for (int i = 1; i < W; ++i) {
        const int dr = (rank + i) % W;
        KNJ_CUDA(cudaMemcpyAsync(c->h_parts[dr] + ((size_t)ch * Tc + (size_t)rank * Tc_loc) * H, stg + (size_t)dr * Tc_loc * H,
                                 (size_t)Tc_loc * H * 4, cudaMemcpyDeviceToDevice, (i & 1) ? side2 : side));
      }
      KNJ_CUDA(cudaEventRecord(c->ev_b, side2));
      KNJ_CUDA(cudaStreamWaitEvent(side, c->ev_b, 0));
    } else {
      KNJ_CUDA(cudaEventRecord(c->ev_down[ch], st));
      KNJ_CUDA(cudaStreamWaitEvent(side, c->ev_down[ch], 0));
      rc = f16p ? ep_combine_partial_peer_f16_at(Y, pe, pw, Tc, H, k, lo, lo + c->e_loc, c->parts_ptrs, (int64_t)ch * Tc * H, rank, Tc_loc, side)
                : ep_combine_partial_peer_at(Y, pe, pw, Tc, H, k, lo, lo + c->e_loc, c->parts_ptrs, (int64_t)ch * Tc * H, nullptr, rank, Tc_loc, side);
      if (rc) return rc;
    }
    KNJ_CUDA(cudaEventRecord(c->ev_sent[ch], side));
    ep_arrive_kernel<<<1, 64, 0, side>>>(c->flag_ptrs, (C + ch) * W, W, rank, epoch);
    rc = launch_status("ep_arrive_kernel");
    if (rc) return rc;
    if (ch >= 1) {
      rc = reduce_chunk(ch - 1);
      if (rc) return rc;
    }
  }
  KNJ_EP_STAMP(7);
  KNJ_CUDA(cudaEventRecord(c->ev_side, side));
  KNJ_CUDA(cudaStreamWaitEvent(st, c->ev_side, 0));  // the caller's stream owns everything the step launched
  KNJ_EP_STAMP(8);
  rc = reduce_chunk(C - 1);
  KNJ_EP_STAMP(9);
  return rc;
}

#ifdef KNJ_TRACE
// measurement builds only: milliseconds between the stamps of the last step (router | - | wait for the first
// chunk's rows | plan | gate+up | down (first chunk) | the remaining chunks | wait for the copy stream | last reduce)
int knj_trace_ep_times(knj_ep_ctx *c, float *ms9) {
  cudaDeviceSynchronize();
  for (int i = 0; i < 9; ++i) cudaEventElapsedTime(ms9 + i, c->stamp[i], c->stamp[i + 1]);
  return 0;
}
#endif

int knj_ep_status(knj_ep_ctx *c, knj_stream_t s) {
  KNJ_REQUIRE(c && c->block, "knj_ep_status: null context");
  int words[2] = {0, 0};
  KNJ_CUDA(cudaMemcpyAsync(words, c->status, sizeof(words), cudaMemcpyDeviceToHost, as_stream(s)));
  KNJ_CUDA(cudaStreamSynchronize(as_stream(s)));
  if (words[0] != 0 || words[1] != 0) {
    set_error("knj_ep: a bounded wait gave up (rank waits %d, GEMMs %d)", words[0], words[1]);
    return KNJ_E_TIMEOUT;
  }
  return KNJ_OK;
}

void knj_ep_destroy(knj_ep_ctx *c) {
  if (!c) return;
  if (c->side) cudaStreamDestroy(c->side);
  if (c->side2) cudaStreamDestroy(c->side2);
  cudaEvent_t evs[5] = {c->ev_fork, c->ev_router, c->ev_side, c->ev_a, c->ev_b};
  for (cudaEvent_t e : evs)
    if (e) cudaEventDestroy(e);
  for (int i = 0; i < KNJ_EP_MAX_CHUNKS; ++i) {
    if (c->ev_down[i]) cudaEventDestroy(c->ev_down[i]);
    if (c->ev_sent[i]) cudaEventDestroy(c->ev_sent[i]);
  }
  if (c->block) cudaFree(c->block);
  delete c;
}

}  // extern "C"
