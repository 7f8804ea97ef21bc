// knj_common.cuh -- shared pieces of the CUDA translation units: status
// plumbing, PTX wrappers (mbarrier, bulk async copy, warp MMA), bounded waits.
#pragma once

#include <cuda.h>
#include <utility>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "knj_device.h"

namespace knj {

// ---- host-side status ------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define KNJ_CUDA(call)                                      \
  do {                                                      \
    cudaError_t e_ = (call);                                \
    if (e_ != cudaSuccess) return ::knj::cuda_fail(e_, #call); \
  } while (0)

#define KNJ_REQUIRE(cond, ...)       \
  do {                               \
    if (!(cond)) {                   \
      ::knj::set_error(__VA_ARGS__); \
      return KNJ_E_REFUSE;           \
    }                                \
  } while (0)

inline int launch_status(const char *what) {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? KNJ_OK : cuda_fail(e, what);
}

inline cudaStream_t as_stream(knj_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int sm_count();  // SMs of the current device (cached per device)
// knj_ep_combine_partial_peer_launch with every owner's array entered at element `parts_off`; with `stage` (f32
// [T][H], local) the rows of other ranks' tokens are written there instead, one dense block per owner
int ep_combine_partial_peer_at(const float *Y, const int32_t *pair_exp, const float *pair_w, int T, int H, int k, int exp_lo, int exp_hi,
                               float *const *parts_ptrs, int64_t parts_off, float *stage, int my_rank, int T_loc, cudaStream_t s);
// the partial rows as fp16 under a per-row power-of-two scale (the slot keeps its f32 stride; H <= 2048, H % 256 == 0),
// and the rank-ordered sum over such slots
int ep_combine_partial_peer_f16_at(const float *Y, const int32_t *pair_exp, const float *pair_w, int T, int H, int k, int exp_lo,
                                   int exp_hi, float *const *parts_ptrs, int64_t parts_off, int my_rank, int T_loc, cudaStream_t s);
int ep_reduce_sel_f16(const float *parts, int n_ranks, int T_loc, int H, const int32_t *pair_exp, int k, int experts_per_rank,
                      const void *resid, int resid_dtype, void *out, int out_dtype, cudaStream_t s);

// Launch of a kernel that belongs to a chain of dependent launches on one stream (the decode layer). With
// overlap on, the launch carries the programmatic-stream-serialization attribute: the grid may be scheduled
// while its predecessor drains, and it must call grid_dep_wait() before it touches anything the predecessor
// wrote. Off (knj_launch_overlap(0)): a plain launch; grid_dep_wait() is then a no-op.
extern int g_chain_overlap;
template <class... KArgs, class... Args>
inline cudaError_t launch_chain(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = g_chain_overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// TMA descriptor over a matrix of `rows` byte rows (`row_bytes` each, a multiple of 16, base 16-byte aligned),
// seen as 32-bit words; one copy moves a box of box_rows rows x box_bytes bytes (box_bytes <= 1024, multiple
// of 16) into dense shared memory. No swizzle; the copy targets this CTA only.
int make_row_tensor_map(CUtensorMap *map, const void *base, uint64_t rows, uint32_t row_bytes, uint32_t box_bytes,
                        uint32_t box_rows);

// Limit (SM clock cycles) of the bounded waits of the decode-class kernels, as set by knj_decode_wait_limit.
long long decode_wait_cycles();

// The cooperative stack launch for the smallest batches (knj_stack_small.cu), behind knj_moe_stack_*.
struct SmallStack;
constexpr int kSmallStackMaxTokens = 2;  // measured: from 3 tokens on the tensor-core kernel is the faster one
int small_stack_create(const knj_moe_ffn_args *layers, int n_layers, SmallStack **out);
int small_stack_launch(SmallStack *st, knj_stream_t s);
int small_stack_status(SmallStack *st, knj_stream_t s);
void small_stack_set_wait(SmallStack *st, long long cycles, int stall);
void small_stack_destroy(SmallStack *st);

// ---- device helpers --------------------------------------------------------
#if defined(__CUDACC__)

// Blocks until the grids this launch depends on have completed and their writes are visible; then lets the
// next launch of the chain be scheduled early. No-ops for a plain launch.
__device__ __forceinline__ void grid_dep_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrival without release ordering: for hand-offs whose data was written to shared memory by the arriving
// warp itself (the same in-order path the arrival takes) and ordered across its lanes by __syncwarp(). A
// releasing arrival would first wait for every asynchronous copy the thread still has in flight.
__device__ __forceinline__ void mbar_arrive_relaxed(uint64_t *bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: every spin in this library gives up after about a second of
// SM clock (2^31 cycles), so a copy or an MMA that never completes cannot hang
// the GPU. Returns false on give-up. `abort_flag` (optional, shared memory) lets
// the threads of a CTA leave together: the first one to give up raises it and
// the others stop waiting as soon as they see it.
constexpr long long kMaxWaitCycles = 1ll << 31;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag = nullptr) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (abort_flag && *abort_flag) return false;
    if (clock64() - t0 > kMaxWaitCycles) {
      if (abort_flag) *abort_flag = 1;
      return false;
    }
  }
}

// The same wait with the limit given at run time (clock cycles).
__device__ __forceinline__ bool mbar_wait_for(uint64_t *bar, uint32_t parity, long long limit_cycles, volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (abort_flag && *abort_flag) return false;
    if (clock64() - t0 > limit_cycles) {
      if (abort_flag) *abort_flag = 1;
      return false;
    }
  }
}

// Same contract, but polls with the non-suspending test_wait: lowest wake-up latency,
// for pipelines whose stage hand-offs sit on the critical path.
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Polling wait with the limit given at run time (clock cycles).
__device__ __forceinline__ bool mbar_spin_for(uint64_t *bar, uint32_t parity, long long limit_cycles, volatile int *abort_flag) {
  if (mbar_test(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_test(bar, parity)) return true;
    if (abort_flag && *abort_flag) return false;
    if (clock64() - t0 > limit_cycles) {
      if (abort_flag) *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_spin(uint64_t *bar, uint32_t parity, volatile int *abort_flag = nullptr) {
  if (mbar_test(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_test(bar, parity)) return true;
    if (abort_flag && *abort_flag) return false;
    if (clock64() - t0 > kMaxWaitCycles) {
      if (abort_flag) *abort_flag = 1;
      return false;
    }
  }
}

// Bulk async copy global -> shared of `bytes` (multiple of 16, both addresses
// 16-byte aligned), completion counted on `bar`. The destination is always this CTA's own shared memory.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// TMA tiled copy of one box: x = first 32-bit word inside the row (a multiple of 4), y = first row.
// Ask for the same box to be brought into L2 only (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_rows(const CUtensorMap *map, int x_words, int y_row) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x_words),
               "r"(y_row)
               : "memory");
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void tma_load_rows(void *dst_smem, const CUtensorMap *map, int x_words, int y_row, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x_words), "r"(y_row), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A * B with a zero accumulator input (lets the compiler feed the zero register
// instead of clearing four registers first)
__device__ __forceinline__ void mma_f16_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float load_as_f32(const void *base, int dtype, int64_t i) {
  if (dtype == KNJ_DT_F32) return static_cast<const float *>(base)[i];
  if (dtype == KNJ_DT_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(base)[i]);
  return __half2float(static_cast<const __half *>(base)[i]);
}
__device__ __forceinline__ void store_from_f32(void *base, int dtype, int64_t i, float v) {
  if (dtype == KNJ_DT_F32) static_cast<float *>(base)[i] = v;
  else if (dtype == KNJ_DT_BF16) static_cast<__nv_bfloat16 *>(base)[i] = __float2bfloat16_rn(v);
  else static_cast<__half *>(base)[i] = __float2half_rn(v);
}

#endif  // __CUDACC__

}  // namespace knj
