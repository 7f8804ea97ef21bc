/* knj_device.h -- C-ABI of libknj_device.so: the device layer and the kernel
 * entry points of the quantized (GGUF Q4_K) MoE expert path, for NVIDIA B200
 * (sm_100a).
 *
 * This is the drop-in boundary. Every entry point replaces one interface of the
 * reference project (cited per declaration as path:line inside that project):
 *   - the HIP runtime calls its drivers make directly (hipMalloc, hipMemcpy,
 *     streams, events) become the thin knj_dev / knj_malloc / knj_stream /
 *     knj_event functions;
 *   - each `extern "C" __global__` kernel becomes a host launcher of the same
 *     name + `_launch`, same arguments in the same order, plus a trailing
 *     stream (a __global__ symbol cannot be launched by a foreign compiler);
 *   - the Q4_K bench kernels' argument lists (the de-facto ExpertPlan) become
 *     knj_q4k_gateup_launch / knj_q4k_proj_launch / knj_q6k_proj_launch /
 *     knj_fuse_gateup_silu_launch (decode class) and knj_q4k_gateup_tc_launch /
 *     knj_q4k_down_tc_launch (prefill class);
 *   - the host routing plan and weighted combine of the benches become device
 *     kernels (knj_router_topk_launch, knj_moe_permute_launch,
 *     knj_moe_combine_launch) and the whole layer is one call
 *     (knj_moe_ffn_decode_launch / knj_moe_ffn_prefill_launch).
 *
 * Conventions.
 *   - Every function returns int: 0 = ok, negative = error (codes below). No
 *     exception crosses this boundary. knj_last_error_string() describes the
 *     last error on the calling thread.
 *   - All buffers are owned by the caller. The kernel launches allocate no
 *     device memory: those that need scratch take an explicit workspace whose
 *     size a *_workspace_bytes function reports. The object constructors do
 *     allocate and say so where they are declared: knj_moe_stack_create (the
 *     stack launch's scratch), knj_ep_create (the rank's private scratch of the
 *     expert-parallel layer), the residency slot pool and the pinned arena
 *     (knj_residency.h). The library image also carries a 64 KiB device array
 *     per GPU, the scratch of knj_q4k_matmul_noalloc_launch.
 *   - Quantized weights are borrowed and immutable: Q4_K superblocks of 144
 *     bytes, row-major [expert][row][K/256][144], base address 16-byte aligned
 *     (KNJ_E_REFUSE otherwise).
 *   - Launches are asynchronous on the given stream (NULL = default stream).
 *     Kernels report nothing themselves: callers that want proof of execution
 *     pre-fill outputs with a sentinel, as the reference's drivers do.
 *   - Thread model: one thread issues launches per stream; the library keeps
 *     no global device state beyond the current device.
 */
#ifndef KNJ_DEVICE_H
#define KNJ_DEVICE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes, mapped onto the reference's failure labels
 * (docs/BUILD-OUTLINE.md:588-598: RETRY / DEGRADE / REFUSE / INVALIDATE / FATAL) */
#define KNJ_OK 0
#define KNJ_E_REFUSE (-1)    /* REFUSE: null pointer, bad geometry, misaligned base */
#define KNJ_E_RUNTIME (-2)   /* FATAL:  a CUDA runtime call failed */
#define KNJ_E_ARCH (-3)      /* REFUSE: device is not compute capability 10.x */
#define KNJ_E_WORKSPACE (-4) /* REFUSE: workspace missing or too small */
#define KNJ_E_TIMEOUT (-5)   /* RETRY:  a bounded device-side wait gave up */
#define KNJ_E_NOTREADY (-6)  /* event / stream query: work still in flight */

/* Process exit codes of the reference's device drivers
 * (tests/test_gemm_w4.hip:11-18, tools/bench/q4k_moe_ffn.hip:63). */
#define KNJ_EXIT_PASS 0
#define KNJ_EXIT_MISSING_INPUT 3
#define KNJ_EXIT_FAIL 5
#define KNJ_EXIT_DECLINED 6 /* built for another arch than the attached device: a skip */
#define KNJ_EXIT_REFUSED 7  /* KNJ_BUILD_ARCH not set */
#define KNJ_EXIT_RUNTIME 9

/* element types of activation buffers */
#define KNJ_DT_F32 0
#define KNJ_DT_BF16 1
#define KNJ_DT_F16 2

typedef void *knj_stream_t; /* a cudaStream_t */
typedef void *knj_event_t;  /* a cudaEvent_t */
typedef void *knj_graph_t;  /* a cudaGraphExec_t */

/* ======================================================================== */
/* Device layer (replaces the hip* calls listed per function)               */
/* ======================================================================== */

/* C mirror of DeviceCaps (src/device/device_caps.h:57-85), runtime fields filled. */
typedef struct knj_device_caps {
  char arch[16]; /* "sm_100" */
  char name[64];
  int32_t has_mma, has_fp8, has_dot_builtin, wave_size;
  uint64_t vram_total, vram_usable;
  int32_t rebar_full_aperture;
  uint32_t sms, clock_khz, max_streams, num_queue_groups;
  uint32_t smem_per_block_optin, l2_bytes;
  int32_t cc_major, cc_minor;
} knj_device_caps;

const char *knj_last_error_string(void);            /* hipGetErrorString(hipGetLastError()) */
int knj_dev_count(int *n);                           /* hipGetDeviceCount */
int knj_dev_open(int idx);                           /* hipSetDevice + arch check; KNJ_E_ARCH if not sm_10x */
int knj_dev_current(int *idx);                       /* hipGetDevice */
int knj_dev_caps(int idx, knj_device_caps *out);     /* hipGetDeviceProperties + hipMemGetInfo */
int knj_dev_sync(void);                              /* hipDeviceSynchronize */
int knj_mem_info(size_t *free_bytes, size_t *total); /* hipMemGetInfo */
/* Arch guard of the drivers (tests/test_gemm_w4.hip:124-142): compares env
 * KNJ_BUILD_ARCH with the compiled arch and the attached device. Returns the
 * driver exit code: 0 ok, 6 declined (mismatch), 7 refused (unset), 9 no device. */
int knj_arch_check(void);

int knj_malloc(void **p, size_t bytes);      /* hipMalloc */
int knj_free(void *p);                       /* hipFree */
int knj_host_malloc(void **p, size_t bytes); /* hipHostMalloc (pinned) */
int knj_host_free(void *p);                  /* hipHostFree */
int knj_memset(void *p, int byte, size_t n, knj_stream_t s); /* hipMemsetAsync */
int knj_memcpy_h2d(void *dst, const void *src, size_t n);    /* hipMemcpy, blocking */
int knj_memcpy_d2h(void *dst, const void *src, size_t n);
int knj_memcpy_d2d(void *dst, const void *src, size_t n);
int knj_memcpy_h2d_async(void *dst, const void *src, size_t n, knj_stream_t s); /* hipMemcpyAsync */
int knj_memcpy_d2h_async(void *dst, const void *src, size_t n, knj_stream_t s);
int knj_memcpy_d2d_async(void *dst, const void *src, size_t n, knj_stream_t s);

int knj_stream_create(knj_stream_t *s); /* hipStreamCreateWithFlags(non-blocking) */
int knj_stream_destroy(knj_stream_t s);
int knj_stream_sync(knj_stream_t s);
int knj_stream_query(knj_stream_t s);                     /* 0 idle, KNJ_E_NOTREADY busy */
int knj_stream_wait_event(knj_stream_t s, knj_event_t e); /* hipStreamWaitEvent */
int knj_event_create(knj_event_t *e, int timing);         /* hipEventCreateWithFlags */
int knj_event_destroy(knj_event_t e);
int knj_event_record(knj_event_t e, knj_stream_t s);
int knj_event_query(knj_event_t e);
int knj_event_sync(knj_event_t e);
int knj_event_elapsed_ms(float *ms, knj_event_t start, knj_event_t stop);

/* Stream capture into a replayable graph (the resident whole-stack loop,
 * tools/bench/q4k_stream_ffn.hip:1233-1325, issues the same launches per step). */
int knj_graph_begin(knj_stream_t s);
int knj_graph_end(knj_stream_t s, knj_graph_t *g);
int knj_graph_launch(knj_graph_t g, knj_stream_t s);
int knj_graph_destroy(knj_graph_t g);

/* ======================================================================== */
/* Kernels of kernels/knj_kernels.hip                                       */
/* ======================================================================== */

/* knj_control (kernels/knj_kernels.hip:132-144): out[0] = seed + 1,
 * out[1] = n_blocks; proves a dispatch happened. */
int knj_control_launch(uint32_t *out, uint32_t seed, uint32_t n_threads, uint32_t n_blocks, knj_stream_t s);

/* knj_probe_caps (kernels/knj_kernels.hip:282-318), launched <<<1,32>>>.
 * cap[0] = dp4a(0x01010101, 0x01010101, 0) == 4; cap[1] = two chained packed
 * half2 fma of 1*1 from zero give 2.0h (0x4000); cap[2] = 1 (dispatched);
 * cap[3] = in ? in[0] : 0; cap[4] = the observed fp16 pattern.
 * CUDA additions: cap[5] = a fp16 tensor-core MMA multiplied subnormal-encoded
 * 4-bit integers exactly (the decode kernels rely on it); cap[6] = a
 * cp.async.bulk + mbarrier transaction completed within its bounded wait;
 * cap[7] = 128 TMEM columns were allocated and freed. cap must hold 8 words. */
int knj_probe_caps_launch(uint32_t *cap, const int32_t *in, knj_stream_t s);

/* knj_build_asum (kernels/knj_kernels.hip:232-260): Asum[m][g] = sum of the
 * 128 int8 activations of group g of row m; Act is [M][K/8][2] u32. */
int knj_build_asum_launch(const uint32_t *Act, int32_t *Asum, uint32_t M, uint32_t K, uint32_t n_threads,
                          uint32_t n_blocks, knj_stream_t s);

/* knj_gemm_w4_i8 (kernels/knj_kernels.hip:176-218): C[m][n] = sum_g scale_g *
 * (sum_k u_k a_k - 8 * Asum[m][g]); Bq is [N][K/128][68]. */
int knj_gemm_w4_i8_launch(const uint8_t *Bq, const uint32_t *Act, const int32_t *Asum, float *C, uint32_t M,
                          uint32_t N, uint32_t K, uint32_t n_threads, uint32_t n_blocks, knj_stream_t s);

/* The dot helpers of include/knj_dot.h on the device (kernels/knj_dot.h:117-174;
 * device mirrors tools/bench/gemm_w4.hip:345-397): out4/out8/out2[i] =
 * knj_dot4_i32_i8 / knj_dot8_i32_i4 / knj_dot2_i32_i16 (a[i], b[i], acc[i]). */
int knj_dot_helpers_launch(const int32_t *a, const int32_t *b, const int32_t *acc, int32_t *out4, int32_t *out8,
                           int32_t *out2, int n, knj_stream_t s);

/* ======================================================================== */
/* Q4_K decode (kernels/knj_q4k.h, src/loader/dequant.cpp)                  */
/* ======================================================================== */

/* Verification kernel: n_blocks Q4_K superblocks -> n_blocks*256 f32, bit-equal
 * to dequant_q4_k (src/loader/dequant.cpp:102-125) and knj_q4k_weight
 * (kernels/knj_q4k.h:147-167). Never on a timed path: the hot kernels fuse the
 * unpack into their consumer. */
int knj_q4k_dequant_launch(const uint8_t *blocks, float *out, uint64_t n_blocks, knj_stream_t s);
/* Same for Q6_K (src/loader/dequant.cpp:164-191, kernels/knj_q4k.h:170-196). */
int knj_q6k_dequant_launch(const uint8_t *blocks, float *out, uint64_t n_blocks, knj_stream_t s);

/* Decode-class projection over Q6_K weights (tools/bench/q4k_stream_ffn.hip:780-829
 * knj_q6k_down with dq4 = 0; CPU dot_q6_k src/loader/dequant.cpp:986-1022):
 * Y[p][n] = sum_k W6[e][n][k] * A[p][k] for the pairs p of every active expert e
 * (tables as for knj_q4k_proj_launch). A f32 [P][K] dense, W6 uint8
 * [E][N][K/256][210] (rows need no alignment; a 16-byte aligned base with N a
 * multiple of 64 takes the bulk-copy staging), Y f32 [P][N]. mma.sync.m16n8k16
 * on exact fp16 codes (q - 32), the activations as two fp16 planes under a
 * power-of-two scale per row (f32-level accuracy), the int8 group scales and d
 * applied in f32. status (optional):
 * set to 1 when a bounded wait for a weight block gave up. */
int knj_q6k_proj_launch(const float *A, const uint8_t *W6, const int32_t *pair_idx, const int32_t *pair_cnt,
                        const int32_t *exp_list, const int32_t *n_active, float *Y, int N, int K, int64_t idxStride,
                        int n_experts, int *status, knj_stream_t s);

/* ======================================================================== */
/* Routing (src/model/model.cpp:419-460; tools/bench/q4k_stream_ffn.hip:957-1001)
 * ======================================================================== */

/* RMSNorm rows (src/model/model.cpp:258-271): out = x * rsqrt(mean(x^2)+eps) * w,
 * w bf16 [H]; out f32 [T][H]. */
int knj_rmsnorm_launch(const void *x, int x_dtype, int64_t ldx, const uint16_t *w_bf16, float eps, int T, int H,
                       float *out, knj_stream_t s);

/* Router: logits[t][e] = x[t] . Wr[e] (+ bias[e]), softmax over E, exact top-k
 * (ties to the lowest expert id), renormalised weights. Pair p = t*k + s holds
 * the s-th most probable expert of token t (the numbering of build_plan).
 * Wr is bf16 [E][H]; bias f32 [E] or NULL; logits f32 [T][E] scratch (also an
 * output); pair_exp int32 [T*k]; pair_w f32 [T*k]. E <= 256, k <= 8. */
int knj_router_topk_launch(const void *x, int x_dtype, int64_t ldx, const uint16_t *Wr_bf16, const float *bias, int T,
                           int H, int E, int k, float *logits, int32_t *pair_exp, float *pair_w, knj_stream_t s);

/* Token permutation: from pair_exp[P] build, per expert, the ascending list of
 * pair ids routed to it -- pair_idx[E][idx_stride] (-1 padded), pair_cnt[E] --
 * plus the ascending list of experts that received work, exp_list[E] with
 * n_active[0] entries used and n_active[1] = max count. Replaces the host loop
 * tools/bench/q4k_moe_ffn.hip:536-548. */
int knj_moe_permute_launch(const int32_t *pair_exp, int P, int E, int idx_stride, int32_t *pair_idx, int32_t *pair_cnt,
                           int32_t *exp_list, int32_t *n_active, knj_stream_t s);

/* The same tables for long pair lists (P >= 8192) by a counting sort that is
 * parallel over the pairs; `scratch` holds knj_moe_permute_scratch_bytes(P, E)
 * bytes. Shorter lists (or scratch == NULL) take knj_moe_permute_launch. */
size_t knj_moe_permute_scratch_bytes(int P, int E);
int knj_moe_permute_ws_launch(const int32_t *pair_exp, int P, int E, int idx_stride, int32_t *pair_idx, int32_t *pair_cnt,
                              int32_t *exp_list, int32_t *n_active, void *scratch, size_t scratch_bytes, knj_stream_t s);

/* Decode front end in one launch (T <= 64): per-row RMSNorm scale (norm_w NULL =
 * none), router logits + softmax + exact top-k (as knj_router_topk_launch over
 * the normalised rows), the permutation tables (as knj_moe_permute_launch) and
 * the normalised rows xn f32 [T][H] the experts see (as knj_rmsnorm_launch).
 * Replaces, for the decode step, rmsnorm_rows + the router part of Model::moe
 * (src/model/model.cpp:631, :419-460) and the host plan of the benches. counter:
 * 64 device words of scratch (the launch zeroes what it uses). H <= 2048, rows of
 * x 16-byte aligned. */
int knj_moe_front_launch(const void *x, int x_dtype, int64_t ldx, const uint16_t *norm_w, float eps,
                         const uint16_t *Wr_bf16, const float *bias, int T, int H, int E, int k, float *logits,
                         int32_t *pair_exp, float *pair_w, int32_t *pair_idx, int idx_stride, int32_t *pair_cnt,
                         int32_t *exp_list, int32_t *n_active, float *xn, uint32_t *counter, knj_stream_t s);

/* Second half of the permutation step alone: exp_list / n_active from pair_cnt. */
int knj_active_list_launch(const int32_t *pair_cnt, int E, int32_t *exp_list, int32_t *n_active, knj_stream_t s);

/* Weighted combine (tools/bench/q4k_moe_ffn.hip:682-694;
 * src/model/model.cpp:502-507): out[t] = (residual ? resid[t] : 0) + sum over
 * the k pairs of token t of pair_w[p] * Y[row_of(p)], summed in ascending
 * expert order as the CPU path does. Y f32 [rows][H]; row_of = pair_row[p] when
 * given, else p. out dtype f32 or bf16. */
int knj_moe_combine_launch(const float *Y, const int32_t *pair_row, const int32_t *pair_exp, const float *pair_w,
                           const void *resid, int resid_dtype, int64_t ld_resid, void *out, int out_dtype, int64_t ldo,
                           int T, int H, int k, knj_stream_t s);

/* ======================================================================== */
/* Expert projections, decode class (f32-accurate, HBM-bound)               */
/* ======================================================================== */

/* The decode kernels multiply Q4_K codes as exact small integers on the fp16
 * tensor cores: a 4-bit code left in place in an fp16 word is an exact subnormal,
 * one packed fp16 multiply folds the 6-bit sub-block scale in, and the activations
 * are split on the fly into a high and a low fp16 plane under a power-of-two scale
 * per (token, 256-wide superblock), ~22 significant bits together. Results agree
 * with the f32 CPU path to <= 1e-5 relative RMSE. Rows of at most 4096 weights.
 * Activation rows (f32, bf16 or f16) must be 16-byte aligned.
 * status (optional device int, zeroed by the caller) is set to 1 if a bounded
 * wait inside the kernel gave up; the outputs are then incomplete. */

/* Gate and up in one pass (tools/bench/q4k_moe_ffn.hip:164-241 knj_q4k_gateup):
 * for every pair p routed to expert e and every n < N
 *   G[p][n] = x[tok(p)] . Wg[e][n],  U[p][n] = x[tok(p)] . Wu[e][n],
 *   A[p][n] = silu(G) * U                       (tools/bench/q4k_stream_ffn.hip:1005-1031)
 * X holds one activation row per TOKEN (row stride ldx elements); tok(p) =
 * pair_tok[p] when given, else p / top_k. G, U, A are f32 [P][N]; any of them may
 * be NULL (not stored). Experts are taken from exp_list[0 .. n_active[0]). */
int knj_q4k_gateup_launch(const void *X, int x_dtype, int64_t ldx, const uint8_t *Wg, const uint8_t *Wu,
                          const int32_t *pair_idx, const int32_t *pair_cnt, const int32_t *pair_tok,
                          const int32_t *exp_list, const int32_t *n_active, float *G, float *U, float *A, int N, int K,
                          int rowBytes, int64_t idxStride, int n_experts, int top_k, int *status, knj_stream_t s);

/* One projection per pair (tools/bench/q4k_stream_ffn.hip:834-882 knj_q4k_proj;
 * :780-829 knj_q6k_down with dq4 = 1): Y[p][n] = a[row(p)] . W[e][n]. A holds
 * one activation row per PAIR (row(p) = pair_row[p] when given, else p; row
 * stride lda elements). Y f32 [P][N]. */
int knj_q4k_proj_launch(const void *A, int a_dtype, int64_t lda, const uint8_t *W, const int32_t *pair_idx,
                        const int32_t *pair_cnt, const int32_t *pair_row, const int32_t *exp_list, const int32_t *n_active,
                        float *Y, int N, int K, int rowBytes, int64_t idxStride, int n_experts, int *status,
                        knj_stream_t s);
#define knj_q4k_down_launch knj_q4k_proj_launch

/* Limit, in SM clock cycles, of every bounded wait of the decode-class kernels
 * (no reference counterpart; default about one second, <= 0 restores it). A wait
 * that runs out makes the kernel skip the rest of its work and raise its status
 * word; nothing traps and the context stays usable. */
void knj_decode_wait_limit(long long cycles);

/* A[i] = silu(G[i]) * U[i], n elements (tools/bench/q4k_stream_ffn.hip:1021-1031
 * knj_fuse_gateup_silu); out dtype f32, bf16 or f16. Uses expf, not the fast
 * intrinsic, so the f32 path keeps its 1e-5 budget. */
int knj_fuse_gateup_silu_launch(const float *G, const float *U, void *A, int a_dtype, int64_t n, knj_stream_t s);

/* Single-matrix GEMV/GEMM convenience (the CPU path's Model::matmul,
 * src/model/model.cpp:326-380): y[m][n_out] = x[m][n_in] . W^T, W Q4_K
 * [n_out][n_in/256][144]. workspace >= knj_q4k_matmul_workspace_bytes(m, n_in). */
size_t knj_q4k_matmul_workspace_bytes(int m, int n_in);
int knj_q4k_matmul_launch(const uint8_t *W, int n_in, int n_out, const void *x, int x_dtype, int64_t ldx, int m,
                          float *y, int64_t ldy, void *workspace, size_t workspace_bytes, knj_stream_t s);

/* Allocation-free form of knj_q4k_matmul_launch. No counterpart in the
 * reference: it exists for callers that may not allocate device memory when
 * they call and have no workspace to lend (a serving loop whose pool is fully
 * committed to resident experts, a plug-in host that only receives input and
 * output buffers, start-up-only allocation policies). Scratch is a fixed array
 * inside the library image, knj_q4k_matmul_noalloc_max_scratch() bytes (64 KiB,
 * enough for 16,256 activation rows),
 * held by every GPU that loads the library until the process exits. Returns
 * KNJ_E_WORKSPACE when knj_q4k_matmul_workspace_bytes(m, n_in) exceeds it. All
 * calls on a device share the array: calls that overlap on the GPU race and must
 * be serialised by the caller. The first call on a device resolves the array's
 * address; make it before any stream capture begins. Calls no allocator. */
size_t knj_q4k_matmul_noalloc_max_scratch(void);
int knj_q4k_matmul_noalloc_launch(const uint8_t *W, int n_in, int n_out, const void *x, int x_dtype, int64_t ldx, int m,
                                  float *y, int64_t ldy, knj_stream_t s);

/* ======================================================================== */
/* Expert projections, prefill class (tcgen05, <= 1e-3)                      */
/* ======================================================================== */

/* x [rows][K] (f32/bf16/f16, row stride ldx) -> dense fp16 [rows][K], values
 * saturated to the fp16 range: the token operand of the grouped GEMMs. */
int knj_to_f16_launch(const void *x, int x_dtype, int64_t ldx, int rows, int K, void *out_f16, knj_stream_t s);

/* 1 = run every bucket of the grouped GEMMs in the single-SM form (tcgen05
 * cta_group::1), the form buckets with an odd number of row tiles always take;
 * 0 (default) = CTA pairs wherever the tile count is even. Process-wide. */
void knj_q4k_tc_single_sm(int on);

/* Launch mode of the kernels of a decode layer (no reference counterpart).
 * 1 (default): programmatic stream serialization -- each grid may be scheduled
 * while its predecessor on the stream drains and waits on the device for the
 * predecessor's completion before reading its results; 0: plain launches. */
void knj_launch_overlap(int on);

/* Grouped gate+up GEMM over per-expert token buckets on the tensor cores
 * (tools/bench/q4k_moe_ffn.hip:164-241 knj_q4k_gateup fused with
 * tools/bench/q4k_stream_ffn.hip:1021-1031 knj_fuse_gateup_silu): for every
 * pair p of expert e, A[p][n] = silu(x[tok(p)].Wg[e][n]) * (x[tok(p)].Wu[e][n]),
 * stored as fp16 scaled by 2^-6 (saturating). Xh fp16 [T][K]; tok(p) =
 * pair_tok[p] when given, else p / top_k. N % 128 == 0. max_pairs bounds the
 * launch grid (the total number of pairs). status (optional device int) is set
 * to 1 if a bounded wait inside the kernel gave up. */
int knj_q4k_gateup_tc_launch(const void *Xh, const uint8_t *Wg, const uint8_t *Wu, const int32_t *pair_idx,
                             const int32_t *pair_cnt, const int32_t *pair_tok, void *A_f16, int N, int K, int rowBytes,
                             int64_t idxStride, int n_experts, int top_k, int max_pairs, int *status, knj_stream_t s);
/* Grouped down GEMM (tools/bench/q4k_stream_ffn.hip:780-829 knj_q6k_down with
 * dq4 = 1): Y[p][n] = 2^6 * (A[row(p)] . Wd[e][n]), A fp16 as written by the
 * gate+up kernel, Y f32 [P][N]; row(p) = pair_row[p] when given, else p. */
int knj_q4k_down_tc_launch(const void *Ah, const uint8_t *Wd, const int32_t *pair_idx, const int32_t *pair_cnt,
                           const int32_t *pair_row, float *Y, int N, int K, int rowBytes, int64_t idxStride,
                           int n_experts, int max_pairs, int *status, knj_stream_t s);

/* Grouped down GEMM over Q6_K weights (tools/bench/q4k_stream_ffn.hip:780-829 knj_q6k_down with dq4 = 0; the
 * mixed-format layers of Q4_K_M files): as knj_q4k_down_tc_launch with W6 [E][N][K/256][210]. The tile's rows are
 * staged whole in shared memory, so K <= 1024. */
int knj_q6k_down_tc_launch(const void *Ah, const uint8_t *W6, const int32_t *pair_idx, const int32_t *pair_cnt,
                           const int32_t *pair_row, float *Y, int N, int K, int64_t idxStride, int n_experts, int max_pairs,
                           int *status, knj_stream_t s);

/* Grouped down GEMM with the weighted scatter-combine in its epilogue (the sum the
 * reference does on the host, tools/bench/q4k_moe_ffn.hip:682-694, residual
 * tools/bench/q4k_stream_ffn.hip:1305-1313): acc[p / top_k][n] += pair_w[p] * 2^6 *
 * (A[row(p)] . Wd[e][n]) for every pair p, as f32 vector reductions in L2. acc f32
 * [T][N] holds the start value (knj_moe_acc_init_launch: the residual rows or zero);
 * knj_moe_acc_finish_launch converts it to the output's element type. No per-pair
 * rows are written. The order of a token's k additions is not fixed. */
int knj_q4k_down_combine_tc_launch(const void *Ah, const uint8_t *Wd, const int32_t *pair_idx, const int32_t *pair_cnt,
                                   const int32_t *pair_row, const float *pair_w, int top_k, float *acc, int N, int K,
                                   int rowBytes, int64_t idxStride, int n_experts, int max_pairs, int *status, knj_stream_t s);
int knj_moe_acc_init_launch(const void *x, int x_dtype, int64_t ldx, int residual, int T, int H, float *acc, knj_stream_t s);
int knj_moe_acc_finish_launch(const float *acc, void *out, int out_dtype, int64_t ldo, int T, int H, knj_stream_t s);

/* ======================================================================== */
/* Whole MoE-FFN layer (src/model/model.cpp:399-510 Model::moe)             */
/* ======================================================================== */

typedef struct knj_moe_ffn_args {
  int32_t n_tokens, hidden, ffn, n_experts, top_k;
  int32_t x_dtype;           /* KNJ_DT_F32 or KNJ_DT_BF16 */
  const void *x;             /* [T][hidden] */
  int64_t ldx;               /* row stride of x, elements */
  const uint16_t *w_router;  /* bf16 [E][hidden] */
  const float *router_bias;  /* f32 [E] or NULL */
  const uint8_t *w_gate;     /* Q4_K [E][ffn][hidden/256][144] */
  const uint8_t *w_up;       /* Q4_K [E][ffn][hidden/256][144] */
  const uint8_t *w_down;     /* Q4_K [E][hidden][ffn/256][144] */
  const uint16_t *norm_w;    /* bf16 [hidden] RMSNorm weight applied to x first, or NULL */
  float rms_eps;
  int32_t residual;          /* 1: out = x + moe(norm(x)); 0: out = moe(norm(x)) */
  void *out;                 /* [T][hidden] */
  int32_t out_dtype;         /* KNJ_DT_F32 or KNJ_DT_BF16 */
  int64_t ldo;
  void *workspace;           /* >= knj_moe_ffn_workspace_bytes(...) */
  size_t workspace_bytes;
  /* optional taps, may be NULL: the routing decision for inspection */
  int32_t *tap_pair_exp;     /* [T*k] */
  float *tap_pair_w;         /* [T*k] */
  /* format of w_down: 0 = Q4_K as above, 1 = Q6_K [E][hidden][ffn/256][210] (the
   * mixed-format layers of Q4_K_M checkpoints; the prefill launch takes them for ffn <= 1024) */
  int32_t down_format;
  /* prefill launch: 0 = per-pair rows + the ordered combine kernel (bit-reproducible, the CPU path's summation
   * order; the faster form on B200 at every measured size); 1 = the weighted combine fused into the down GEMM's
   * epilogue as f32 vector reductions in L2 (no per-pair rows are written; the k rows of a token are added in
   * no fixed order, so results vary in the last bits between runs) */
  int32_t fused_combine;
} knj_moe_ffn_args;

/* mode 0 = decode class (knj_moe_ffn_decode_launch), 1 = prefill class. */
size_t knj_moe_ffn_workspace_bytes(int n_tokens, int hidden, int ffn, int n_experts, int top_k, int mode);

/* Decode: batch <= 64 tokens, HBM-bound, f32-accurate (<= 1e-5 rel-RMSE vs the
 * CPU path). Larger T is accepted and stays exact, at decode-class speed. */
int knj_moe_ffn_decode_launch(const knj_moe_ffn_args *a, knj_stream_t s);
/* Prefill: tokens bucketed per expert, Q4_K unpacked to fp16 operands for
 * tcgen05.mma with f32 TMEM accumulators (<= 1e-3 rel-RMSE vs the CPU path). */
int knj_moe_ffn_prefill_launch(const knj_moe_ffn_args *a, knj_stream_t s);
/* Outcome of the last layer launch over this argument block (same workspace):
 * waits for the stream, then KNJ_OK, or KNJ_E_TIMEOUT when a bounded wait inside
 * one of its kernels gave up (docs/BUILD-OUTLINE.md:588-598: RETRY). mode as for
 * knj_moe_ffn_workspace_bytes. */
int knj_moe_ffn_status(const knj_moe_ffn_args *a, int mode, knj_stream_t s);

/* The resident decode stack for a decode batch of 1..64 tokens in ONE cooperative
 * launch: n_layers layer descriptions (layer l's out is normally layer l+1's x; out
 * must not alias x within a layer), all of one shape; a layer's down matrices are
 * Q4_K or Q6_K (down_format, per layer: the mixed-format stacks of Q4_K_M files). The loop
 * the reference runs on the host per layer (src/model/model.cpp:399-510) becomes
 * grid barriers inside one kernel. Same arithmetic class as
 * knj_moe_ffn_decode_launch (f32, <= 1e-5 rel-RMSE vs the CPU path; routing
 * decisions identical to it). create validates, builds the layer table on the
 * device and ALLOCATES the launch's scratch (cudaMalloc; freed by destroy); the
 * workspace fields of the layer descriptions are not used. status() waits for the
 * stream and returns KNJ_E_TIMEOUT when a bounded wait inside the kernel (a grid
 * barrier or a weight copy) gave up. One launch of a stack may be in flight at a
 * time (its barrier words are per stack), and the launch needs every SM of the
 * device (cooperative launch, one CTA per SM). */
typedef struct knj_moe_stack knj_moe_stack;
int knj_moe_stack_create(const knj_moe_ffn_args *layers, int n_layers, knj_moe_stack **out);
int knj_moe_stack_decode_launch(knj_moe_stack *st, knj_stream_t s);
int knj_moe_stack_status(knj_moe_stack *st, knj_stream_t s);
/* Limit of the kernel's bounded waits in SM clock cycles (<= 0: the default, about
 * a second), and a fault-injection hook for tests of the RETRY path
 * (docs/BUILD-OUTLINE.md:588-598): stall_first_barrier > 0 raises the first grid
 * barrier's target by that many arrivals, so the wait runs out, every CTA returns
 * and status() reports KNJ_E_TIMEOUT; 0 restores normal operation. Nothing traps
 * and the context stays usable. */
int knj_moe_stack_set_wait(knj_moe_stack *st, long long wait_cycles, int stall_first_barrier);
void knj_moe_stack_destroy(knj_moe_stack *st);

/* ======================================================================== */
/* Device-clock spans for a host profiler                                   */
/* ======================================================================== */
/* The event ring behind Profiler::device_span(name, start_ns, end_ns, stream)
 * (src/profiler/profiler.h:98-137): spans are offsets from ONE epoch event on the
 * stream, handed over at flush time, never inside the step loop; spans the ring
 * could not hold are counted. While recording is on, knj_moe_ffn_decode_launch
 * and knj_moe_ffn_prefill_launch bracket their stages with spans named as the
 * CPU path's rows (src/model/model.cpp:408-500): moe-router, moe-gather,
 * moe-gate (gate + up + activation, fused), moe-down, moe-scatter. Nothing is
 * recorded on a stream that is being captured into a graph. One recorder per
 * process; not thread-safe. */
int knj_spans_enable(int capacity);            /* (re)starts recording with room for `capacity` spans */
int knj_spans_disable(void);
int knj_spans_active(void);                     /* 1 while recording is on */
int knj_spans_epoch(knj_stream_t s);            /* marks time zero on `s`, empties the ring */
int knj_span_begin(const char *name, knj_stream_t s);   /* handle >= 0, or -1: not recorded */
int knj_span_end(int handle, knj_stream_t s);
uint64_t knj_spans_dropped(void);               /* spans refused since the epoch because the ring was full */
/* Waits for the recorded events, then calls cb(name, start_ns, end_ns, 0, user)
 * for every closed span in recording order, and empties the ring. */
int knj_spans_flush(void (*cb)(const char *name, uint64_t start_ns, uint64_t end_ns, int stream, void *user), void *user);

/* ======================================================================== */
/* Expert-parallel exchange helpers                                         */
/* ======================================================================== */
/* The reference keeps every expert on one device and has no counterpart for
 * these two (multi-GPU is a declared non-goal there, README.md:104-107,
 * docs/01-architecture.md:322-325). Experts are split contiguously over ranks,
 * owner(e) = e / (E / n_ranks). The all-to-all itself is issued by the host
 * (NCCL); these kernels prepare and consume its buffers.
 *
 * knj_ep_pack: copy the hidden row of every pair (row_bytes each, token =
 * pair / top_k) into send_rows in (expert, pair) order -- which is also
 * destination-rank order -- and record pair_row[p] = slot of pair p, the index
 * the combine uses on the returned rows. send_off[E+1] receives the exclusive
 * scan of pair_cnt. */
int knj_ep_pack_launch(const void *x, int row_bytes, int top_k, const int32_t *pair_idx, int idx_stride,
                       const int32_t *pair_cnt, int E, int32_t *send_off, void *send_rows, int32_t *pair_row,
                       knj_stream_t s);
/* knj_ep_plan: counts[r][e] = rows source rank r sent for local expert e (rows
 * of one source are contiguous, experts ascending). Builds the local plan over
 * received-row indices: pair_idx[E_loc][idx_stride], pair_cnt, exp_list,
 * n_active, as knj_moe_permute_launch does for local pairs. */
int knj_ep_plan_launch(const int32_t *counts, int n_ranks, int n_local_experts, int idx_stride, int32_t *pair_idx,
                       int32_t *pair_cnt, int32_t *exp_list, int32_t *n_active, knj_stream_t s);

/* Gather exchange, step 1 (no reference counterpart; the partial form of the
 * weighted sum at src/model/model.cpp:455-463): out[t][:] = sum over the pairs of
 * token t whose expert id lies in [exp_lo, exp_hi), ascending expert id, of
 * pair_w * Y[pair][:], separately rounded multiply and add from zero; zeros for
 * tokens without such a pair. Y rows are indexed by pair id t*k+s. out f32 [T][H]. */
int knj_ep_combine_partial_launch(const float *Y, const int32_t *pair_exp, const float *pair_w, int T, int H, int k,
                                  int exp_lo, int exp_hi, float *out, knj_stream_t s);

/* Gather exchange, step 2: out[t][:] = (resid[t][:] +) sum over ranks r = 0..n_ranks-1
 * (ascending) of parts[r*rank_stride + t*H + :]; out f32 or bf16, dense rows. */
int knj_ep_reduce_launch(const float *parts, int n_ranks, int64_t rank_stride, int T, int H, const void *resid,
                         int resid_dtype, void *out, int out_dtype, knj_stream_t s);

/* Peer exchange (no reference counterpart): the gather exchange with the rows
 * moved by this library's kernels over NVLink peer mappings instead of NCCL
 * collectives. src_ptrs / parts_ptrs are DEVICE arrays of n_ranks pointers, entry
 * r = rank r's exchange buffer mapped into this process (entry own-rank = the
 * local buffer). The caller orders the steps across ranks (a barrier after the
 * rows are published and one after the partial rows are stored).
 * knj_ep_peer_gather: dst[r*bytes_per_rank + i] = src_ptrs[r][i].
 * knj_ep_combine_partial_peer: as knj_ep_combine_partial, but the row of token t
 * goes to parts_ptrs[t / T_loc][(my_rank*T_loc + t % T_loc)*H ...] and tokens
 * without an expert in [exp_lo, exp_hi) are skipped.
 * knj_ep_reduce_sel: out[t] = (resid[t] +) sum, ascending rank r, of
 * parts[(r*T_loc + t)*H ...] over the ranks that own one of token t's k experts
 * (rank of expert e = e / experts_per_rank); pair_exp is the LOCAL table [T_loc*k]. */
int knj_ep_peer_gather_launch(const void *const *src_ptrs, int n_ranks, int64_t bytes_per_rank, void *dst, knj_stream_t s);
int knj_ep_combine_partial_peer_launch(const float *Y, const int32_t *pair_exp, const float *pair_w, int T, int H, int k,
                                       int exp_lo, int exp_hi, float *const *parts_ptrs, int my_rank, int T_loc,
                                       knj_stream_t s);
int knj_ep_reduce_sel_launch(const float *parts, int n_ranks, int T_loc, int H, const int32_t *pair_exp, int k,
                             int experts_per_rank, const void *resid, int resid_dtype, void *out, int out_dtype,
                             knj_stream_t s);

/* ---------------------------------------------------------------------------
 * The expert-parallel layer of one rank as one object (no reference counterpart;
 * the per-rank arithmetic is src/model/model.cpp:399-510). One process per GPU;
 * the five exchange buffers of EVERY rank are mapped into this process (CUDA IPC,
 * symmetric memory or any other peer mapping made by the host) and passed as HOST
 * arrays of `world` device pointers, entry r = rank r's buffer, entry `rank` =
 * this rank's own:
 *   xall_ptrs  fp16 [world*n_tokens_local][hidden]  every rank's rows
 *   pe_ptrs    int32 [world*n_tokens_local*top_k]   every rank's expert ids
 *   pw_ptrs    f32   [world*n_tokens_local*top_k]   every rank's routing weights
 *   parts_ptrs f32   [world][n_tokens_local][hidden] partial sums of this rank's tokens, by contributing rank
 *   flag_ptrs  uint32 [KNJ_EP_FLAG_WORDS]            flag words, zero before the first step
 * knj_ep_create allocates the rank's private scratch (plan tables, the activation
 * and per-pair output rows) once; knj_ep_forward_launch allocates nothing and calls
 * no collective library. A step runs in n_chunks chunks of the local tokens
 * (chunk c = local tokens [c, c+1) * n_tokens_local / n_chunks of EVERY rank; the
 * gathered buffers are chunk-major: rows [n_chunks][world][chunk tokens][hidden],
 * likewise the tables and the partial sums) over the caller's stream and a copy
 * stream of the context:
 *   copy streams: per chunk the rank's rows (fp16) and routing tables are written
 *                 into every rank's buffers, then an arrival word into every rank's
 *                 flags; later the chunk's weighted partial sums go to the token
 *                 owners the same way
 *   caller's    : router over the local tokens; per chunk: wait until every rank's
 *                 arrival word is there (bounded spin; a wait that gives up raises
 *                 the status word read by knj_ep_status -> KNJ_E_TIMEOUT and the
 *                 step's output is then undefined), plan, the grouped tensor-core
 *                 GEMMs over the rank's experts, and -- one chunk behind -- the
 *                 rank-ordered sum of the partial rows (+ residual = x)
 * so that a chunk's transfers overlap the neighbouring chunks' GEMMs. When the
 * call returns the caller's stream is ordered after everything it launched.
 * All ranks must call knj_ep_forward_launch the same number of times (the flag
 * words carry the step number).
 * hidden, ffn multiples of 256; (n_tokens_local / n_chunks) * top_k a multiple of
 * 4; experts split contiguously, n_experts / world <= 256; n_chunks 0 or 1 = one.
 * ------------------------------------------------------------------------- */
#define KNJ_EP_COPY_ENGINES 0 /* rows and partial sums travel as block copies (one cudaMemcpyAsync per peer) */
#define KNJ_EP_SM_ROWS 1      /* the rows travel as 16-byte stores of this library's kernels */
#define KNJ_EP_SM_PARTIALS 2  /* the partial sums travel as 16-byte stores of the kernel that forms them */
#define KNJ_EP_F16_PARTIALS 4 /* with KNJ_EP_SM_PARTIALS, hidden <= 2048: the partial rows travel as fp16 under a per-row
                                 power-of-two scale (half the bytes; 2^-11 relative to the row's largest element) */
#define KNJ_EP_FLAG_WORDS 4096
#define KNJ_EP_MAX_CHUNKS 8
typedef struct knj_ep_desc {
  int32_t world, rank, n_tokens_local, hidden, ffn, n_experts, top_k, n_chunks;
  void *const *xall_ptrs;
  int32_t *const *pe_ptrs;
  float *const *pw_ptrs;
  float *const *parts_ptrs;
  uint32_t *const *flag_ptrs;
} knj_ep_desc;
typedef struct knj_ep_ctx knj_ep_ctx;
int knj_ep_create(const knj_ep_desc *desc, knj_ep_ctx **out);
/* w_router bf16 [n_experts][hidden] (replicated), router_bias f32 [n_experts] or NULL;
 * w_gate / w_up / w_down: this rank's experts, Q4_K, [n_experts/world][rows][row bytes].
 * x [n_tokens_local][ldx] f32 / bf16 / fp16; out dense f32 or bf16 [n_tokens_local][hidden]. */
int knj_ep_forward_launch(knj_ep_ctx *ctx, const void *x, int x_dtype, int64_t ldx, const uint16_t *w_router,
                          const float *router_bias, const uint8_t *w_gate, const uint8_t *w_up, const uint8_t *w_down,
                          int residual, void *out, int out_dtype, knj_stream_t s);
/* a barrier over the ranks on the stream (arrival + bounded wait in one launch, on flag words of its own) */
int knj_ep_barrier_launch(knj_ep_ctx *ctx, knj_stream_t s);
/* How rows and partial sums reach the peers: an OR of KNJ_EP_SM_ROWS, KNJ_EP_SM_PARTIALS and KNJ_EP_F16_PARTIALS,
 * 0 = block copies for both (the routing tables and the flag words always go as stores of the library's kernels). With block copies the
 * SMs stay with the GEMMs while a chunk travels; partial sums then travel as dense blocks per owner, rows of tokens
 * without an expert on the sender included (never read). Default KNJ_EP_SM_PARTIALS | KNJ_EP_F16_PARTIALS: block copies
 * for the rows, the partial sums stored by the kernel that forms them (only contributing rows travel) as fp16 under
 * a per-row power-of-two scale -- the sums themselves are formed and added in f32; the stored form costs about
 * 1e-4 relative RMSE of the layer output, inside the 1e-3 budget of the tensor-core path. Without the flag the rows
 * travel as f32 and the result equals the single-GPU layer's to ~5e-8. Every rank must use the same transport. */
int knj_ep_set_transport(knj_ep_ctx *ctx, int transport);
/* limit of every rank wait in SM clock cycles (<= 0 restores the default, about a second) */
int knj_ep_set_wait(knj_ep_ctx *ctx, long long wait_cycles);
/* synchronises the stream; KNJ_E_TIMEOUT if a barrier or a GEMM pipeline wait gave up since the last step began */
int knj_ep_status(knj_ep_ctx *ctx, knj_stream_t s);
void knj_ep_destroy(knj_ep_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* KNJ_DEVICE_H */
