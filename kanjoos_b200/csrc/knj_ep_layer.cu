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
// slot `rank` of j's flag array) and waits until rank j has told this rank the same (slot j of the own array).
// Everything this rank stored into peer memory before the launch is visible to a peer that leaves its barrier.
// A wait that runs out of time raises *status and the kernel returns; nothing spins without a limit.
__global__ void ep_barrier_kernel(uint32_t *const *flags, int world, int rank, uint32_t *epoch, long long limit, int *status) {
  const int j = threadIdx.x;
  const uint32_t e = *epoch + 1u;
  __threadfence_system();
  if (j < world) {
    st_release_sys(flags[j] + rank, e);
    const uint32_t *mine = flags[rank] + j;
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

// The rank's rows as fp16 into every rank's gathered-rows buffer at row offset rank * T_loc (16 bytes = 8 values
// per thread and step, one store per destination).
template <int DT>
__global__ void __launch_bounds__(256) ep_push_rows_kernel(const void *__restrict__ x, int64_t ldx, int H8, int64_t n8,
                                                           __half *const *__restrict__ dst, int world, int64_t dst_off) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / H8, c = 8 * (i - r * H8);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = load_as_f32(x, DT, r * ldx + c + j);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 h = __floats2half2_rn(fminf(fmaxf(v[2 * j], -65504.0f), 65504.0f), fminf(fmaxf(v[2 * j + 1], -65504.0f), 65504.0f));
      o[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
    const uint4 u = make_uint4(o[0], o[1], o[2], o[3]);
    for (int d = 0; d < world; ++d) *reinterpret_cast<uint4 *>(dst[d] + dst_off + r * (int64_t)H8 * 8 + c) = u;
  }
}

// The rank's slice of the routing tables from its own gathered tables to the peers' (16 bytes per thread).
__global__ void __launch_bounds__(256) ep_push_tables_kernel(int32_t *const *__restrict__ pe, float *const *__restrict__ pw, int world,
                                                             int rank, int64_t off, int64_t n4) {
  const uint4 *spe = reinterpret_cast<const uint4 *>(pe[rank] + off), *spw = reinterpret_cast<const uint4 *>(pw[rank] + off);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 a = spe[i], b = spw[i];
    for (int d = 0; d < world; ++d) {
      if (d == rank) continue;
      reinterpret_cast<uint4 *>(pe[d] + off)[i] = a;
      reinterpret_cast<uint4 *>(pw[d] + off)[i] = b;
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
  int T = 0, P = 0, e_loc = 0;
  char *block = nullptr;  // one device allocation, carved below
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
  // local scratch
  float *logits = nullptr, *Y = nullptr;
  int32_t *local_ids = nullptr, *pair_idx = nullptr, *pair_cnt = nullptr, *exp_list = nullptr, *n_active = nullptr;
  void *perm_scratch = nullptr, *ah = nullptr;
  size_t perm_bytes = 0;
  uint32_t *epoch = nullptr;
  int *status = nullptr;  // [0] barrier, [1] GEMMs
  long long wait_cycles = kMaxWaitCycles;
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
};

extern "C" {

int knj_ep_create(const knj_ep_desc *desc, knj_ep_ctx **out) {
  KNJ_REQUIRE(desc && out, "knj_ep_create: null argument");
  *out = nullptr;
  const knj_ep_desc &d = *desc;
  KNJ_REQUIRE(d.world >= 1 && d.world <= 64 && d.rank >= 0 && d.rank < d.world, "knj_ep_create: rank %d of %d", d.rank, d.world);
  KNJ_REQUIRE(d.n_experts >= d.world && d.n_experts % d.world == 0 && d.n_experts / d.world <= 256,
              "knj_ep_create: %d experts do not split over %d ranks", d.n_experts, d.world);
  KNJ_REQUIRE(d.n_tokens_local >= 1 && d.hidden % 256 == 0 && d.ffn % 256 == 0 && d.hidden % 128 == 0 && d.ffn % 128 == 0,
              "knj_ep_create: bad token count / hidden / ffn");
  KNJ_REQUIRE(d.top_k >= 1 && d.top_k <= 8 && ((int64_t)d.n_tokens_local * d.top_k) % 4 == 0,
              "knj_ep_create: top_k out of range or local pairs not a multiple of 4");
  KNJ_REQUIRE(d.xall_ptrs && d.pe_ptrs && d.pw_ptrs && d.parts_ptrs && d.flag_ptrs, "knj_ep_create: null pointer table");
  for (int r = 0; r < d.world; ++r)
    KNJ_REQUIRE(d.xall_ptrs[r] && d.pe_ptrs[r] && d.pw_ptrs[r] && d.parts_ptrs[r] && d.flag_ptrs[r] && aligned16(d.xall_ptrs[r]) &&
                    aligned16(d.pe_ptrs[r]) && aligned16(d.pw_ptrs[r]) && aligned16(d.parts_ptrs[r]),
                "knj_ep_create: rank %d's buffers are missing or not 16-byte aligned", r);
  knj_ep_ctx *c = new knj_ep_ctx();
  c->d = d;
  c->T = d.n_tokens_local * d.world;
  c->P = c->T * d.top_k;
  c->e_loc = d.n_experts / d.world;
  const size_t T = c->T, P = c->P, H = d.hidden, F = d.ffn, W = d.world;
  c->perm_bytes = knj_moe_permute_scratch_bytes(c->P, c->e_loc);
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t at = off; off += up256(bytes); return at; };
  const size_t o_tab = take(5 * W * sizeof(void *));
  const size_t o_logits = take((size_t)d.n_tokens_local * d.n_experts * 4);
  const size_t o_ids = take(P * 4);
  const size_t o_pidx = take((size_t)c->e_loc * T * 4);
  const size_t o_small = take((size_t)(2 * c->e_loc + 16) * 4);
  const size_t o_perm = take(c->perm_bytes);
  const size_t o_ah = take(P * F * 2);
  const size_t o_y = take(P * H * 4);
  const size_t o_words = take(64);
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&c->block), off);
  if (e == cudaSuccess) e = cudaMemset(c->block + o_words, 0, 64);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming);
  void **tab = reinterpret_cast<void **>(c->block + o_tab);
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
  c->logits = reinterpret_cast<float *>(c->block + o_logits);
  c->local_ids = reinterpret_cast<int32_t *>(c->block + o_ids);
  c->pair_idx = reinterpret_cast<int32_t *>(c->block + o_pidx);
  c->pair_cnt = reinterpret_cast<int32_t *>(c->block + o_small);
  c->exp_list = c->pair_cnt + c->e_loc;
  c->n_active = c->exp_list + c->e_loc;
  c->perm_scratch = c->block + o_perm;
  c->ah = c->block + o_ah;
  c->Y = reinterpret_cast<float *>(c->block + o_y);
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

int knj_ep_barrier_launch(knj_ep_ctx *c, knj_stream_t s) {
  KNJ_REQUIRE(c && c->block, "knj_ep_barrier: null context");
  ep_barrier_kernel<<<1, 64, 0, as_stream(s)>>>(c->flag_ptrs, c->d.world, c->d.rank, c->epoch, c->wait_cycles, c->status);
  return launch_status("ep_barrier_kernel");
}

int knj_ep_forward_launch(knj_ep_ctx *c, const void *x, int x_dtype, int64_t ldx, const uint16_t *w_router,
                          const float *router_bias, const uint8_t *w_gate, const uint8_t *w_up, const uint8_t *w_down,
                          int residual, void *out, int out_dtype, knj_stream_t s) {
  KNJ_REQUIRE(c && c->block && x && w_router && w_gate && w_up && w_down && out, "knj_ep_forward: null pointer");
  KNJ_REQUIRE(x_dtype == KNJ_DT_F32 || x_dtype == KNJ_DT_BF16 || x_dtype == KNJ_DT_F16, "knj_ep_forward: unknown x dtype");
  KNJ_REQUIRE(out_dtype == KNJ_DT_F32 || out_dtype == KNJ_DT_BF16, "knj_ep_forward: out must be f32 or bf16");
  const knj_ep_desc &d = c->d;
  const int T_loc = d.n_tokens_local, H = d.hidden, F = d.ffn, k = d.top_k, W = d.world, rank = d.rank, T = c->T, P = c->P;
  KNJ_REQUIRE(ldx >= H && ldx % 8 == 0 && aligned16(x), "knj_ep_forward: rows of x must be 16-byte aligned");
  cudaStream_t st = as_stream(s);
  int rc;
  // ---- rows to every rank (side stream) while the router runs (main stream)
  KNJ_CUDA(cudaEventRecord(c->ev_fork, st));
  KNJ_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
  {
    const int64_t n8 = (int64_t)T_loc * H / 8, blocks = (n8 + 255) / 256, cap = (int64_t)sm_count() * 4;
    const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
    const int64_t off = (int64_t)rank * T_loc * H;
    if (x_dtype == KNJ_DT_F32) ep_push_rows_kernel<KNJ_DT_F32><<<grid, 256, 0, c->side>>>(x, ldx, H / 8, n8, c->xall_ptrs, W, off);
    else if (x_dtype == KNJ_DT_BF16) ep_push_rows_kernel<KNJ_DT_BF16><<<grid, 256, 0, c->side>>>(x, ldx, H / 8, n8, c->xall_ptrs, W, off);
    else ep_push_rows_kernel<KNJ_DT_F16><<<grid, 256, 0, c->side>>>(x, ldx, H / 8, n8, c->xall_ptrs, W, off);
    rc = launch_status("ep_push_rows_kernel");
    if (rc) return rc;
    KNJ_CUDA(cudaEventRecord(c->ev_join, c->side));
  }
  KNJ_CUDA(cudaMemsetAsync(c->status, 0, 2 * sizeof(int), st));
  const int64_t toff = (int64_t)rank * T_loc * k;
  rc = knj_router_topk_launch(x, x_dtype, ldx, w_router, router_bias, T_loc, H, d.n_experts, k, c->logits, c->pe_all + toff,
                              c->pw_all + toff, s);
  if (rc) return rc;
  if (W > 1) {
    const int64_t n4 = (int64_t)T_loc * k / 4;
    ep_push_tables_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(c->pe_ptrs, c->pw_ptrs, W, rank, toff, n4);
    rc = launch_status("ep_push_tables_kernel");
    if (rc) return rc;
  }
  KNJ_CUDA(cudaStreamWaitEvent(st, c->ev_join, 0));
  rc = knj_ep_barrier_launch(c, s);  // every rank's rows and tables have landed here
  if (rc) return rc;
  // ---- this rank's experts over all tokens
  const int lo = rank * c->e_loc;
  ep_local_ids_kernel<<<(unsigned)((P + 255) / 256 < 1184 ? (P + 255) / 256 : 1184), 256, 0, st>>>(c->pe_all, lo, c->e_loc, P, c->local_ids);
  rc = launch_status("ep_local_ids_kernel");
  if (rc) return rc;
  rc = knj_moe_permute_ws_launch(c->local_ids, P, c->e_loc, T, c->pair_idx, c->pair_cnt, c->exp_list, c->n_active, c->perm_scratch,
                                 c->perm_bytes, s);
  if (rc) return rc;
  rc = knj_q4k_gateup_tc_launch(c->x_all, w_gate, w_up, c->pair_idx, c->pair_cnt, nullptr, c->ah, F, H, H / 256 * KNJ_Q4K_BYTES, T,
                                c->e_loc, k, P, c->status + 1, s);
  if (rc) return rc;
  rc = knj_q4k_down_tc_launch(c->ah, w_down, c->pair_idx, c->pair_cnt, nullptr, c->Y, H, F, F / 256 * KNJ_Q4K_BYTES, T, c->e_loc, P,
                              c->status + 1, s);
  if (rc) return rc;
  // ---- weighted partial sums to the token owners, then the sum over the contributing ranks
  rc = knj_ep_combine_partial_peer_launch(c->Y, c->pe_all, c->pw_all, T, H, k, lo, lo + c->e_loc, c->parts_ptrs, rank, T_loc, s);
  if (rc) return rc;
  rc = knj_ep_barrier_launch(c, s);
  if (rc) return rc;
  return knj_ep_reduce_sel_launch(c->parts, W, T_loc, H, c->pe_all + toff, k, c->e_loc, residual ? x : nullptr, x_dtype, out, out_dtype, s);
}

int knj_ep_status(knj_ep_ctx *c, knj_stream_t s) {
  KNJ_REQUIRE(c && c->block, "knj_ep_status: null context");
  int words[2] = {0, 0};
  KNJ_CUDA(cudaMemcpyAsync(words, c->status, sizeof(words), cudaMemcpyDeviceToHost, as_stream(s)));
  KNJ_CUDA(cudaStreamSynchronize(as_stream(s)));
  if (words[0] != 0 || words[1] != 0) {
    set_error("knj_ep: a bounded wait gave up (rank barrier %d, GEMMs %d)", words[0], words[1]);
    return KNJ_E_TIMEOUT;
  }
  return KNJ_OK;
}

void knj_ep_destroy(knj_ep_ctx *c) {
  if (!c) return;
  if (c->side) cudaStreamDestroy(c->side);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  if (c->block) cudaFree(c->block);
  delete c;
}

}  // extern "C"
