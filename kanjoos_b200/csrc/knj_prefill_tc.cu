// knj_prefill_tc.cu -- prefill-class grouped expert GEMM on the 5th-generation
// tensor cores: Q4_K weights are unpacked to fp16 in shared memory and consumed
// by tcgen05.mma with f32 accumulators in tensor memory.
//
// Roles (swap-AB): the MMA "M" side is weight rows of one expert, the "N" side is
// a bucket of up to 256 routed tokens (a multiple of 16), K runs over the hidden
// (or ffn) dimension in slabs of 64 (one 128-byte swizzle row of fp16). Per CTA
// one (expert, 128-row tile, token bucket); where a bucket has an even number of
// row tiles, CTAs 2i and 2i+1 form a cluster and share one cta_group::2 MMA
// (M = 256 over the pair, each CTA gathers half of the bucket's token rows):
//   warps 0..7  unpackers: 2-D TMA boxes (32 rows x 144 B) bring the raw
//               superblocks into a double-buffered staging area; per superblock
//               the eight (d*sc, -dmin*m) pairs are formed in fp16 (exact), per
//               slab each thread turns 16 code bytes into 32 fp16 weights and
//               stores them into the K-major 128-byte-swizzled operand tile
//               (three operand stages);
//   warp 8      one elected thread issues tcgen05.mma (kind::f16) over the four
//               16-wide steps of a slab and commits the stage back to the
//               producers; in a pair the even CTA issues for both and its commit
//               arrives on the barriers of both CTAs (tcgen05.commit with the
//               multicast::cluster qualifier: a barrier arrival, no data moves);
//   warps 9..12 loaders: gather the token rows of the slab with 16-byte cp.async
//               straight into the swizzled tile; completion arrives on the stage
//               barrier (cp.async.mbarrier.arrive.noinc), so several slabs are in
//               flight with no registers held;
//   warps 0..7  epilogue: tcgen05.ld of the accumulators (lane = weight row,
//               column = token), SiLU(gate)*up or the plain projection (or the
//               weighted reduction into the token's sum), transposed through the
//               idle operand stages, 16-byte row stores.
// Gate and up share the token operand: two accumulators (TMEM columns [0,256)
// and [256,512)) are fed from two weight tiles per slab.
//
// Precision. Operands are fp16, not bf16: a Q4_K weight rounded to fp16 is off
// by <= 2^-12 relative, which keeps the layer's relative RMSE well inside the
// 1e-3 budget of the tensor-core path; bf16 operands (2^-9) would not. The
// activations are converted to fp16 beforehand with a saturating convert, and
// the SiLU*up intermediate is stored as fp16 after a fixed 2^-6 prescale
// (undone in the down epilogue), which holds magnitudes up to 4.1e6.
//
// Every wait on an mbarrier is bounded; on give-up the kernel raises a status
// flag, still frees its tensor memory and returns.
#include "knj_common.cuh"
#include "knj_q4k.h"

using namespace knj;

namespace {

constexpr int kRowsM = 128;        // weight rows per tile and CTA (MMA M per CTA)
constexpr int kMaxTok = 256;       // token bucket (MMA N upper bound)
constexpr int kSlabK = 64;         // K elements per pipeline stage (one 128-byte swizzle row)
constexpr int kProducerThreads = 256;  // unpacker warps 0..7
constexpr int kLoaderThreads = 128;    // loader warps 9..12
constexpr int kThreads = kProducerThreads + 32 + kLoaderThreads;
constexpr float kActPrescale = 0.015625f;  // 2^-6

struct TcParams {
  const __half *X;        // activation rows, fp16 [rows][K]
  const uint8_t *W0;      // gate or the single matrix, Q4_K [E][N][K/256][144]
  const uint8_t *W1;      // up (dual) or null
  const int32_t *pair_idx;
  const int32_t *pair_cnt;
  const int32_t *row_map;  // pair -> activation row (null: pair / row_div)
  void *out;               // dual: fp16 act [P][N]; single: f32 Y [P][N]
  int N, K, rowBytes, row_div, n_experts, m_tiles;
  int64_t idxStride;
  float out_scale;
  int *status;
  // fused weighted combine (single-matrix form only; cmb_acc == null: off): instead of storing the per-pair row,
  // the epilogue adds cmb_w[pair] * row into cmb_acc[pair / cmb_div] with vector reductions in L2
  const float *cmb_w;
  float *cmb_acc;
  int cmb_div;
#ifdef KNJ_TRACE
  unsigned long long *trace;  // measurement builds: SM-clock stamps of CTA 0's first slabs
  int trace_ctas;             // per-CTA records that fit behind the 64 slab stamps
#endif
  CUtensorMap map0, map1;     // TMA descriptors of W0 / W1, box = one superblock (36 words) x 32 rows
};

#ifdef KNJ_TRACE
unsigned long long *g_tc_trace = nullptr;
int g_tc_trace_ctas = 0;
#define KNJ_TC_STAMP(cond, slot)              \
  do {                                        \
    if (p.trace && (cond)) p.trace[slot] = clock64(); \
  } while (0)
#define KNJ_TC_SET_TRACE(p) ((p).trace = g_tc_trace, (p).trace_ctas = g_tc_trace_ctas)
#else
#define KNJ_TC_STAMP(cond, slot) ((void)0)
#define KNJ_TC_SET_TRACE(p) ((void)0)
#endif
int g_tc_force_single = 0;  // 1 = never pair CTAs (knj_q4k_tc_single_sm)

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Every tcgen05 instruction of one kernel names the same CTA group: CG = 1 (one SM per tile) or 2 (a pair of
// CTAs of one cluster works on one 256-row tile: each brings its own 128 weight rows and half of the tokens).
template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t *slot_smem, uint32_t ncols) {
  if (CG == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "r"(ncols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
  if (CG == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if (CG == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// the barrier (a shared::cluster address: this CTA's or the peer's) gets one arrival once every MMA issued so far
// has completed
template <int CG>
__device__ __forceinline__ void tc_commit_addr(uint32_t bar_addr) {
  if (CG == 1) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
  else asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
// the same, signalled to the barrier at this shared-memory offset in both CTAs of the pair by one instruction
// (a barrier arrival, not a data copy)
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_addr) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar_addr),
               "h"(mask)
               : "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t cluster_addr(const void *smem_ptr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(smem_ptr)), "r"(rank));
  return r;
}
// arrive on a barrier given by its shared::cluster address (this CTA's or the peer's). The data it publishes
// is read by the tensor core through the async proxy, ordered by the writer's fence.proxy.async.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
// 16-byte asynchronous copy global -> shared (L2 only); src_bytes = 0 writes zeros
__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(src_bytes) : "memory");
}
// one arrival on the barrier once every cp.async this thread has issued so far has landed
__device__ __forceinline__ void cp_async_arrive(uint64_t *bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// all threads of both CTAs of the pair
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// D(tmem) (+)= A(smem desc) * B(smem desc), fp16 operands, f32 accumulate
template <int CG>
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  const uint32_t zero = 0;
  if (CG == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(zero), "r"(zero), "r"(zero), "r"(zero)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(zero), "r"(zero), "r"(zero), "r"(zero),
          "r"(zero), "r"(zero), "r"(zero), "r"(zero)
        : "memory");
}
// 16 consecutive f32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// K-major, 128-byte swizzle, rows of 64 fp16 (128 bytes), 8-row groups 1024
// bytes apart: start address, LBO (unused for swizzled K-major) = 1, SBO = 64
// (1024 >> 4), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)64 << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor: D = f32, A = B = f16, both K-major, M = 128 per CTA of the group
__device__ __forceinline__ uint32_t instr_desc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// the two unpacker warps that own the same 32 weight rows (one per 16-byte half) meet on their own barrier
__device__ __forceinline__ void pair_sync(int pair) { asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory"); }

constexpr int kQ6MaxSb = 4;  // Q6_K form: superblocks per weight row that the whole-tile staging holds (K <= 1024)

template <int NMAT, int CG, int FMT = 0>
struct Smem {
  // operand tiles: 1024-byte aligned for the swizzle pattern
  static constexpr int kStages = CG == 2 ? 3 : 2;   // operand stages (weights and token rows advance together)
  static constexpr int kStagesA = kStages, kStagesB = kStages;
  static constexpr int kTokCta = kMaxTok / CG;   // token rows this CTA stages per slab
  static constexpr int kATile = kRowsM * 128;    // 16 KB per matrix per stage
  static constexpr int kBTile = kTokCta * 128;   // 32 KB (16 KB in a pair) per stage
  // raw weights: Q4_K two buffers of one superblock per row; Q6_K the tile's rows whole, once (its 210-byte
  // superblocks cannot be fetched as boxes: rows are only 2-byte aligned)
  static constexpr int kRawBuf = FMT == 1 ? kRowsM * kQ6MaxSb * KNJ_Q6K_BYTES : NMAT * kRowsM * KNJ_Q4K_BYTES;
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kOffA + kStagesA * NMAT * kATile;
  static constexpr int kOffRaw = kOffB + kStagesB * kBTile;
  static constexpr int kOffPairs = kOffRaw + (FMT == 1 ? kRawBuf : 2 * kRawBuf);  // int32 pair id per token of the bucket
  static constexpr int kOffRows = kOffPairs + kMaxTok * 4;      // int32 activation row per token
  static constexpr int kOffBars = kOffRows + kMaxTok * 4;       // mbarriers
  static constexpr int kBytes = kOffBars + 256 + 1024;          // + alignment slack
};

// sixteen bytes from a 2-byte aligned shared-memory address as four words: five aligned words, shifted by two
// bytes where the address is odd in units of two (the word past the sixteen bytes is read but, when the address
// is aligned, not used; callers keep it inside their own data)
__device__ __forceinline__ void lds16_u16(const uint8_t *p, uint32_t (&w)[4]) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
  const uint32_t sel = (a & 2) ? 0x5432u : 0x3210u;
  uint32_t v[5];
#pragma unroll
  for (int i = 0; i < 5; ++i) v[i] = q[i];
#pragma unroll
  for (int i = 0; i < 4; ++i) w[i] = __byte_perm(v[i], v[i + 1], sel);
}

// NMAT = 2 with GATEUP: gate and up tiles of the same 128 output indices (one shared token operand, SiLU*up
// epilogue). NMAT = 2 without: two consecutive 128-row tiles of one matrix (halves the token-operand traffic
// of the down projection). NMAT = 1: one tile.
// CG = 2: CTAs 2i and 2i+1 of the grid form a cluster and run tcgen05.mma.cta_group::2 (M = 256 over the pair):
// each CTA unpacks its own weight tiles and stages half of the bucket's token rows, so the token operand
// crosses L2 -> shared memory once per 256 weight rows instead of once per 128. The even CTA issues the MMAs;
// producers of both CTAs arrive on its "full" barriers, and it commits to the "empty" barriers of both.
// FMT = 1: the weights are Q6_K (single matrix, NMAT = 1): the tile's 128 rows are staged whole with 16-byte loads
// by the unpackers themselves and decoded per slab (w = d * sc * (q - 32), formed in fp16 as (1024 + q - 1056) *
// fp16(d * sc)); everything downstream of the operand tile is the Q4_K form's.
template <int NMAT, bool GATEUP, int CG, int FMT = 0>
__global__ void __launch_bounds__(kThreads, 1) q4k_grouped_tc_kernel(const __grid_constant__ TcParams p) {
  static_assert(FMT == 0 || (NMAT == 1 && !GATEUP), "the Q6_K form is the single-matrix projection");
  using S = Smem<NMAT, CG, FMT>;
  constexpr int kStages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = CG == 2 ? cluster_rank() : 0u;  // == blockIdx.x & 1 (m_tiles is even when CG == 2)

  // ---- which (expert, token bucket) is this CTA's? scan the counts (E <= 256)
  const int m_tile = blockIdx.x % p.m_tiles;
  // every warp finds it for itself: lane l holds the counts of experts 8l..8l+7, a warp scan over the bucket
  // counts locates the expert (a serial walk over up to 128 counts cost the late CTAs 2-3 us)
  const int want = blockIdx.x / p.m_tiles;
  int e = -1, tok0 = 0, cnt = 0;
  {
    int cnts[8], nb = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = lane * 8 + j;
      cnts[j] = i < p.n_experts ? p.pair_cnt[i] : 0;
      nb += (cnts[j] + kMaxTok - 1) / kMaxTok;
    }
    int incl = nb;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int excl = incl - nb;
    int fe = -1, ft = 0, fc = 0;
    if (want >= excl && want < incl) {
      int w = want - excl;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int nt = (cnts[j] + kMaxTok - 1) / kMaxTok;
        if (fe < 0) {
          if (w < nt) { fe = lane * 8 + j; ft = w * kMaxTok; fc = cnts[j]; }
          else w -= nt;
        }
      }
    }
    const unsigned owner = __ballot_sync(0xffffffffu, fe >= 0);
    if (owner) {
      const int src = __ffs(owner) - 1;
      e = __shfl_sync(0xffffffffu, fe, src);
      tok0 = __shfl_sync(0xffffffffu, ft, src);
      cnt = __shfl_sync(0xffffffffu, fc, src);
    }
  }
  if (e < 0) return;  // the same for both CTAs of a pair: nothing allocated yet, no barrier touched
#ifdef KNJ_TRACE
  unsigned long long *cta_rec = (p.trace && (int)blockIdx.x < p.trace_ctas) ? p.trace + 256 + 4 * (size_t)blockIdx.x : nullptr;
  if (cta_rec && tid == 0) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    cta_rec[0] = global_timer_ns();
    cta_rec[3] = ((unsigned long long)smid << 32) | (unsigned)(cnt - tok0 < kMaxTok ? cnt - tok0 : kMaxTok);
  }
#define KNJ_TC_REC(i)                                   \
  do {                                                  \
    if (cta_rec && tid == 0) cta_rec[i] = global_timer_ns(); \
  } while (0)
#else
#define KNJ_TC_REC(i) ((void)0)
#endif
  const int ntok = min(kMaxTok, cnt - tok0);
  const int n_mma = (ntok + 15) & ~15;  // MMA N: multiple of 16
  const int n_cta = n_mma / CG;         // token rows staged by this CTA: [rank * n_cta, (rank + 1) * n_cta)
  const int m0 = m_tile * kRowsM * (GATEUP ? 1 : NMAT);
  const int nsb = p.K / KNJ_QK_K, nslab = p.K / kSlabK;

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::kOffBars);
  uint64_t *full = bars;                           // [kStages] unpackers + loaders -> MMA (the even CTA's are used)
  uint64_t *empty = full + kStages;                // [kStages] MMA -> unpackers and loaders
  uint64_t *locB = empty + kStages;                // [kStages] odd CTA only: its own loaders' copies landed
  uint64_t *raw_full = locB + kStages;             // [2 buffers][4 row groups] TMA boxes landed
  uint64_t *acc_full = raw_full + 8;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
  volatile int *s_fail = reinterpret_cast<volatile int *>(tmem_slot + 1);  // raised by the first wait that gives up
  int32_t *s_pair = reinterpret_cast<int32_t *>(smem + S::kOffPairs);
  int32_t *s_row = reinterpret_cast<int32_t *>(smem + S::kOffRows);

  if (tid == 0) {
    // one "full" barrier per stage: 8 unpacker warps per CTA, this CTA's loader threads (asynchronous-copy
    // arrivals) and, in a pair, one relayed arrival for the odd CTA's loaders
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], CG * 8 + kLoaderThreads + (CG == 2 ? 1 : 0));
      mbar_init(&empty[s], 1);
      mbar_init(&locB[s], kLoaderThreads);
    }
    for (int i = 0; i < 8; ++i) mbar_init(&raw_full[i], 1);
    mbar_init(acc_full, 1);
    *s_fail = 0;
    if (CG == 2) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    else mbar_init_fence();
    if (FMT == 1) {
      // Q6_K: the tile's 128 rows are contiguous in HBM and start on a 16-byte boundary (tiles start at multiples
      // of 128 rows, 32 rows are a multiple of 16 bytes): four bulk copies, one per 32-row group, each on its own
      // barrier, under way while the rest of the prologue runs
      const uint32_t grp = 32u * (uint32_t)(p.K / KNJ_QK_K) * KNJ_Q6K_BYTES;
      const uint8_t *src = p.W0 + ((size_t)e * p.N + m_tile * kRowsM) * (size_t)(grp / 32u);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        mbar_expect_tx(&raw_full[g], grp);
        bulk_g2s(smem + S::kOffRaw + g * grp, src + (size_t)g * grp, grp, &raw_full[g]);
      }
    }
  }
  for (int i = tid; i < kMaxTok; i += kThreads) {
    int pr = -1, rw = -1;
    if (i < ntok) {
      pr = p.pair_idx[(size_t)e * p.idxStride + tok0 + i];
      rw = p.row_map ? p.row_map[pr] : pr / p.row_div;
    }
    s_pair[i] = pr;
    s_row[i] = rw;
  }
  constexpr uint32_t kTmemCols = NMAT == 2 ? 512 : 256;
  if (warp == 8) {
    tmem_alloc<CG>(tmem_slot, kTmemCols);
    tmem_relinquish<CG>();
  }
  tc_fence_before();
  __syncthreads();
  if (CG == 2) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;  // once false this thread skips all work and waits but still meets every barrier

  if (FMT == 1 && warp < 8) {
    // =========================== producers, Q6_K ===========================
    const int row = tid & 127, half = tid >> 7;  // weight row, which 16 of a quadrant's 32 weights
    const int row_bytes = nsb * KNJ_Q6K_BYTES;
    uint8_t *rawq = smem + S::kOffRaw;
    if (!mbar_wait(&raw_full[warp & 3], 0, s_fail)) ok = false;  // this warp's 32 rows have landed
    const uint8_t *rrow = rawq + (size_t)row * row_bytes;
    const __half2 k1056 = __float2half2_rn(1056.0f);  // 1024 (the byte-to-fp16 trick) + 32 (the code's offset)
    for (int ks = 0; ks < nslab; ++ks) {
      if (*s_fail) ok = false;
      if (!ok) break;
      const int stage = ks % kStages;
      if (ks >= kStages && !mbar_wait(&empty[stage], ((ks / kStages) - 1) & 1, s_fail)) { ok = false; break; }
      tc_fence_after();
      const int sl = ks & 3, hf = sl >> 1;
      const uint8_t *blk = rrow + (ks >> 2) * KNJ_Q6K_BYTES;
      const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(blk + 208)));
      uint32_t qh[4];
      lds16_u16(blk + 128 + 32 * hf + 16 * half, qh);
      uint8_t *at = smem + S::kOffA + stage * S::kATile + row * 128;
#pragma unroll
      for (int par = 0; par < 2; ++par) {
        const int c = 2 * (sl & 1) + par;  // quadrant of the 128-weight half: weights 32 c + l, l = 16 half + [0, 16)
        uint32_t ql[4];
        lds16_u16(blk + 64 * hf + 32 * par + 16 * half, ql);
        const float sc = (float)reinterpret_cast<const int8_t *>(blk)[192 + 8 * hf + half + 2 * c];
        const __half2 ds = __float2half2_rn(d * sc);
        uint32_t o[8];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint32_t nib = ((sl & 1) ? (ql[w] >> 4) : ql[w]) & 0x0f0f0f0fu;
          const uint32_t q4 = nib | (((qh[w] >> (2 * c)) & 0x03030303u) << 4);
          const uint32_t e01 = __byte_perm(q4, 0x64646464u, 0x4140);
          const uint32_t e23 = __byte_perm(q4, 0x64646464u, 0x4342);
          const __half2 h01 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&e01), k1056), ds);
          const __half2 h23 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&e23), k1056), ds);
          o[2 * w] = *reinterpret_cast<const uint32_t *>(&h01);
          o[2 * w + 1] = *reinterpret_cast<const uint32_t *>(&h23);
        }
        const int c0 = 4 * par + 2 * half;
        *reinterpret_cast<uint4 *>(at + (((c0) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4 *>(at + (((c0 + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        if (CG == 2) mbar_arrive_cluster(cluster_addr(&full[stage], 0));
        else mbar_arrive(&full[stage]);
      }
    }
  } else if (warp < 8) {
    // =========================== producers ===========================
    const int row = tid & 127, half = tid >> 7;  // weight row, which 16 of the slab's 32 code bytes
    const int pair = warp & 3;                   // rows 32*pair .. 32*pair+31: this warp and warp ^ 4
    // one TMA box per matrix and row group: 32 rows x one superblock (a single copy instruction each; per-row
    // bulk copies cost the copy unit about 25 cycles apiece and stalled every superblock boundary)
    auto issue_raw = [&](int b) {
      if (warp < 4 && lane == 0) {
        uint64_t *bar = &raw_full[(b & 1) * 4 + pair];
        mbar_expect_tx(bar, (uint32_t)NMAT * 32u * KNJ_Q4K_BYTES);
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
          uint8_t *dst = smem + S::kOffRaw + (b & 1) * S::kRawBuf + (mat * kRowsM + 32 * pair) * KNJ_Q4K_BYTES;
          const int y = e * p.N + m0 + (GATEUP ? 0 : mat * kRowsM) + 32 * pair;
          tma_load_rows(dst, (GATEUP && mat == 1) ? &p.map1 : &p.map0, b * (KNJ_Q4K_BYTES / 4), y, bar);
        }
      }
    };
    fence_proxy_async();
    issue_raw(0);
    for (int b = 0; b < nsb; ++b) {
      // both warps of the row group are done reading the buffer the next superblock lands in
      pair_sync(pair);
      if (*s_fail) ok = false;
      if (!ok) continue;
      if (b + 1 < nsb) {
        fence_proxy_async();
        issue_raw(b + 1);
      }
      if (!mbar_wait(&raw_full[(b & 1) * 4 + pair], (b >> 1) & 1, s_fail)) { ok = false; continue; }
      const uint8_t *raw = smem + S::kOffRaw + (b & 1) * S::kRawBuf;

      // ---- once per superblock: (d*sc, -dmin*m) of this row's eight sub-blocks in fp16.
      // d*sc is an 11-bit by 6-bit product, so one fp16 multiply rounds it exactly as a
      // float multiply followed by a conversion would.
      const __half2 k1024 = __float2half2_rn(1024.0f);
      __half2 d1h[NMAT][8], m1h[NMAT][8];
#pragma unroll
      for (int mat = 0; mat < NMAT; ++mat) {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(raw + (mat * kRowsM + row) * KNJ_Q4K_BYTES);
        const __half2 dd = __half2half2(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
        const __half2 dm = __hneg2(__half2half2(__ushort_as_half((unsigned short)(hdr.x >> 16))));
        const uint32_t sc4[2] = {hdr.y & 0x3f3f3f3fu, (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u)};
        const uint32_t mn4[2] = {hdr.z & 0x3f3f3f3fu, ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u)};
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
            // bytes (2pr, 2pr+1) of the four six-bit values -> fp16 pair via 1024 + v
            const uint32_t es = __byte_perm(sc4[hb], 0x64646464u, pr ? 0x4342 : 0x4140);
            const uint32_t em = __byte_perm(mn4[hb], 0x64646464u, pr ? 0x4342 : 0x4140);
            const __half2 s2 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&es), k1024), dd);
            const __half2 m2 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&em), k1024), dm);
            d1h[mat][4 * hb + 2 * pr] = __low2half2(s2);
            d1h[mat][4 * hb + 2 * pr + 1] = __high2half2(s2);
            m1h[mat][4 * hb + 2 * pr] = __low2half2(m2);
            m1h[mat][4 * hb + 2 * pr + 1] = __high2half2(m2);
          }
        }
      }

#pragma unroll
      for (int G = 0; G < 4; ++G) {
        if (!ok) break;
        const int ks = b * 4 + G, stage = ks % kStages;
        KNJ_TC_STAMP(blockIdx.x == 0 && tid == 0 && ks < 12, 4 * ks + 0);
        if (ks >= kStages && !mbar_wait(&empty[stage], ((ks / kStages) - 1) & 1, s_fail)) { ok = false; break; }
        tc_fence_after();
        KNJ_TC_STAMP(blockIdx.x == 0 && tid == 0 && ks < 12, 4 * ks + 1);
        // ---- weight operand(s): 16 code bytes -> 16 low-nibble + 16 high-nibble weights of this row
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
          const uint4 q = *reinterpret_cast<const uint4 *>(raw + (mat * kRowsM + row) * KNJ_Q4K_BYTES + KNJ_Q4K_OFF_QS + 32 * G + 16 * half);
          uint8_t *at = smem + S::kOffA + (stage * NMAT + mat) * S::kATile + row * 128;
          const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int par = 0; par < 2; ++par) {
            const __half2 d1 = d1h[mat][2 * G + par], m1 = m1h[mat][2 * G + par];
            uint32_t o[8];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              // the four codes of this word as bytes, then pairs (k0,k1), (k2,k3) as fp16 1024+q
              const uint32_t nib = (par ? (qw[w] >> 4) : qw[w]) & 0x0f0f0f0fu;
              const uint32_t e01 = __byte_perm(nib, 0x64646464u, 0x4140);
              const uint32_t e23 = __byte_perm(nib, 0x64646464u, 0x4342);
              const __half2 h01 = __hfma2(__hsub2(*reinterpret_cast<const __half2 *>(&e01), k1024), d1, m1);
              const __half2 h23 = __hfma2(__hsub2(*reinterpret_cast<const __half2 *>(&e23), k1024), d1, m1);
              o[2 * w] = *reinterpret_cast<const uint32_t *>(&h01);
              o[2 * w + 1] = *reinterpret_cast<const uint32_t *>(&h23);
            }
            // 16 weights = two 16-byte chunks: k_local = 32*par + 16*half + [0,16)
            const int c0 = 4 * par + 2 * half;
            *reinterpret_cast<uint4 *>(at + (((c0) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4 *>(at + (((c0 + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          if (CG == 2) mbar_arrive_cluster(cluster_addr(&full[stage], 0));
          else mbar_arrive(&full[stage]);
        }
        KNJ_TC_STAMP(blockIdx.x == 0 && tid == 0 && ks < 12, 4 * ks + 2);
      }
    }
  } else if (warp >= 9) {
    // =========================== loaders ===========================
    // rows of 64 fp16 per slab; 16-byte chunk c of row r lands at chunk c ^ (r & 7). Asynchronous copies:
    // nothing waits for the gathered rows in registers, so as many slabs travel as there are stages, and
    // the stage's barrier gets this thread's arrival when its copies have landed. (A register path would
    // stall on the release fence of every hand-off until its prefetched loads return.) In a pair each CTA
    // gathers half of the bucket's rows.
    constexpr int kRpt = S::kTokCta / 16;  // rows per thread and slab
    const int lt = tid - (kProducerThreads + 32);
    const int c = lt & 7, r0 = lt >> 3;  // 16 rows per pass
    const __half *rowp[kRpt];
#pragma unroll
    for (int j = 0; j < kRpt; ++j) {
      const int r = r0 + 16 * j;
      const int xr = r < n_cta ? s_row[rank * n_cta + r] : -1;
      rowp[j] = xr >= 0 ? p.X + (size_t)xr * p.K + c * 8 : nullptr;
    }
    for (int ks = 0; ks < nslab && ok; ++ks) {  // loaders meet no CTA barrier before the final one
      const int stage = ks % kStages;
      [[maybe_unused]] const bool ltr = blockIdx.x == 0 && lt == 0 && ks < 12;
      KNJ_TC_STAMP(ltr, 64 + 4 * ks);
      if (ks >= kStages && !mbar_wait(&empty[stage], ((ks / kStages) - 1) & 1, s_fail)) { ok = false; break; }
      KNJ_TC_STAMP(ltr, 64 + 4 * ks + 1);
      uint8_t *bt = smem + S::kOffB + stage * S::kBTile;
#pragma unroll
      for (int j = 0; j < kRpt; ++j) {
        const int r = r0 + 16 * j;
        if (r < n_cta)
          cp_async16(bt + r * 128 + ((c ^ (r & 7)) << 4), rowp[j] ? (const void *)(rowp[j] + ks * kSlabK) : (const void *)p.X,
                     rowp[j] ? 16u : 0u);
      }
      cp_async_arrive(rank == 0 ? &full[stage] : &locB[stage]);
      KNJ_TC_STAMP(ltr, 64 + 4 * ks + 3);
    }
  } else if (CG == 2 && warp == 8 && lane == 0 && rank == 1) {
    // =========================== relay (odd CTA) ===========================
    // cp.async completions can only arrive on a barrier of their own CTA: pass them on to the MMA thread
    for (int ks = 0; ks < nslab && ok; ++ks) {
      const int sb = ks % kStages;
      if (!mbar_spin(&locB[sb], (ks / kStages) & 1, s_fail)) { ok = false; break; }
      mbar_arrive_cluster(cluster_addr(&full[sb], 0));
    }
  } else if (warp == 8 && lane == 0 && rank == 0) {
    // =========================== MMA issue ===========================
    // Every instruction this thread issues (MMA, commit, barrier test) costs it on the order of a hundred
    // cycles, and the tensor pipe queues little: what is not an MMA here is idle pipe time. Hence one "full"
    // barrier per stage for both operands and one commit per CTA.
    const uint32_t idesc = instr_desc_f16(kRowsM * CG, n_mma);
    for (int ks = 0; ks < nslab && ok; ++ks) {
      const int st = ks % kStages;
      if (!mbar_spin(&full[st], (ks / kStages) & 1, s_fail)) { ok = false; break; }
      // No proxy fence here: the unpackers fence their own stores before arriving, the gathered rows are
      // complete when their copies' arrivals are (the hand-off CUTLASS' cp.async tcgen05 main loop relies on),
      // and a fence.proxy.async in this thread would wait for the shared-memory reads of every MMA in flight.
      tc_fence_after();
      KNJ_TC_STAMP(blockIdx.x == 0 && ks < 12, 4 * ks + 3);
      const uint32_t b_addr = smem_u32(smem + S::kOffB + st * S::kBTile);
      const uint32_t a_addr = smem_u32(smem + S::kOffA + st * NMAT * S::kATile);
#pragma unroll
      for (int k = 0; k < kSlabK / 16; ++k) {
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat)  // consecutive instructions alternate between the two accumulators
          tc_mma_f16<CG>(tmem_base + mat * kMaxTok, smem_desc_sw128(a_addr + mat * S::kATile + k * 32),
                         smem_desc_sw128(b_addr + k * 32), idesc, (ks > 0 || k > 0) ? 1u : 0u);
      }
      if (CG == 2) tc_commit_pair(smem_u32(&empty[st]));
      else tc_commit_addr<CG>(smem_u32(&empty[st]));
      KNJ_TC_STAMP(blockIdx.x == 0 && ks < 12, 128 + ks);
    }
    if (ok) {
      if (CG == 2) tc_commit_pair(smem_u32(acc_full));
      else tc_commit_addr<CG>(smem_u32(acc_full));
    }
  }

  // =========================== epilogue ===========================
  if (warp != 8) {
    // unpackers and loaders alike (12 warps); warp w may read the 32 TMEM lanes 32 * (w % 4)
    constexpr int kEpiWarps = 12;
    const int ew = warp < 8 ? warp : warp - 1;          // 0..11
    const int slot = warp < 8 ? (warp >> 2) : 2;        // which of the three warps of a lane group
    if (ok && !mbar_wait(acc_full, 0, s_fail)) ok = false;
    tc_fence_after();
    KNJ_TC_REC(1);
    // The accumulator rows are output indices (one per thread) and the columns tokens, while the outputs are
    // token-major: transpose through the operand stages (idle now), then write whole 256- or 512-byte row
    // segments, 16 bytes per lane. Every unpacker thread takes part in the barriers even after a failed wait.
    [[maybe_unused]] const bool tr = blockIdx.x == 0 && tid == 0;
    KNJ_TC_STAMP(tr, 48);
    const int lane_base = 32 * (warp & 3);
    uint8_t *stg = smem + S::kOffA;
    constexpr int kEpiMats = GATEUP ? 1 : NMAT;
    constexpr int kRowB = GATEUP ? kRowsM * 2 : kRowsM * 4;  // staged bytes per token
    static_assert(kMaxTok * kRowB <= S::kOffPairs, "epilogue staging does not fit the operand stages");
#pragma unroll 1
    for (int mat = 0; mat < kEpiMats; ++mat) {
      if (ok) {
        for (int c = slot; c * 16 < n_mma; c += 3) {
          float g[16];
          tmem_ld16(tmem_base + ((uint32_t)lane_base << 16) + mat * kMaxTok + c * 16, g);
          if (GATEUP) {
            float u[16];
            tmem_ld16(tmem_base + ((uint32_t)lane_base << 16) + kMaxTok + c * 16, u);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              // fast division: the IEEE one takes its slow path whenever exp(-g) overflows
              const float a = __fdividef(g[j], 1.0f + __expf(-g[j])) * u[j] * p.out_scale;
              *reinterpret_cast<__half *>(stg + (c * 16 + j) * kRowB + (lane_base + lane) * 2) =
                  __float2half_rn(fminf(fmaxf(a, -65504.0f), 65504.0f));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              *reinterpret_cast<float *>(stg + (c * 16 + j) * kRowB + (lane_base + lane) * 4) = g[j] * p.out_scale;
          }
        }
      }
      KNJ_TC_STAMP(tr, 49 + 2 * mat);
      asm volatile("bar.sync 5, 384;" ::: "memory");
      if (ok) {
        constexpr int kLanesPerRow = kRowB / 16;            // 16 (fp16) or 32 (f32)
        constexpr int kRowsPerInstr = 32 / kLanesPerRow;    // 2 or 1
        const int sub = lane / kLanesPerRow, l16 = lane % kLanesPerRow;
        for (int r = ew * kRowsPerInstr + sub; r < ntok; r += kEpiWarps * kRowsPerInstr) {
          const int pr = s_pair[r];
          const uint4 v = *reinterpret_cast<const uint4 *>(stg + r * kRowB + l16 * 16);
          if (!GATEUP && p.cmb_acc) {
            // the row's share of its token's weighted sum: one 16-byte reduction per lane (the k rows of a token
            // arrive from different CTAs in no fixed order)
            const float w = __ldg(p.cmb_w + pr);
            float *dst = p.cmb_acc + (size_t)(pr / p.cmb_div) * p.N + m0 + mat * kRowsM + l16 * 4;
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(v.x) * w),
                         "f"(__uint_as_float(v.y) * w), "f"(__uint_as_float(v.z) * w), "f"(__uint_as_float(v.w) * w)
                         : "memory");
            continue;
          }
          uint8_t *dst = GATEUP ? reinterpret_cast<uint8_t *>(static_cast<__half *>(p.out) + (size_t)pr * p.N + m0)
                                : reinterpret_cast<uint8_t *>(static_cast<float *>(p.out) + (size_t)pr * p.N + m0 + mat * kRowsM);
          *reinterpret_cast<uint4 *>(dst + l16 * 16) = v;
        }
      }
      KNJ_TC_STAMP(tr, 50 + 2 * mat);
      if (mat + 1 < kEpiMats) asm volatile("bar.sync 5, 384;" ::: "memory");
    }
  }
  if (!ok && lane == 0 && p.status) atomicExch(p.status, 1);
  tc_fence_before();
  __syncthreads();
  // a CTA of a pair may neither free tensor memory nor leave while the peer still reads its accumulators'
  // operands or arrives on its barriers
  if (CG == 2) cluster_sync_all();
  if (warp == 8) tmem_dealloc<CG>(tmem_base, kTmemCols);
  KNJ_TC_REC(2);
}

// x (f32 / bf16 / f16) -> fp16 with saturation, rows dense
__global__ void to_f16_kernel(const void *__restrict__ x, int dtype, int64_t ldx, int K, int64_t n, __half *__restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / K, c = i - r * K;
    const float v = load_as_f32(x, dtype, r * ldx + c);
    out[i] = __float2half_rn(fminf(fmaxf(v, -65504.0f), 65504.0f));
  }
}

// the common case, bf16 rows whose length and stride are multiples of 8: 16 bytes in, 16 bytes out per thread and step
__global__ void __launch_bounds__(256) bf16_to_f16_kernel(const uint4 *__restrict__ x, int64_t ldx8, int K8, int64_t n8,
                                                          uint4 *__restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / K8, c = i - r * K8;
    const uint4 v = __ldg(x + r * ldx8 + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
      const __half2 h = __floats2half2_rn(fminf(fmaxf(lo, -65504.0f), 65504.0f), fminf(fmaxf(hi, -65504.0f), 65504.0f));
      o[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// acc[t][:] = residual ? x[t][:] : 0 (f32), the start value of the fused weighted combine; four columns per thread
__global__ void __launch_bounds__(256) acc_init_kernel(const void *__restrict__ x, int dtype, int64_t ldx, int residual, int H,
                                                       int64_t n4, float *__restrict__ acc) {
  const int H4 = H / 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (residual) {
      const int64_t t = i / H4, c = 4 * (i - t * H4);
      v.x = load_as_f32(x, dtype, t * ldx + c);
      v.y = load_as_f32(x, dtype, t * ldx + c + 1);
      v.z = load_as_f32(x, dtype, t * ldx + c + 2);
      v.w = load_as_f32(x, dtype, t * ldx + c + 3);
    }
    reinterpret_cast<float4 *>(acc)[i] = v;
  }
}
// out[t][:] = acc[t][:] in the output's element type
__global__ void __launch_bounds__(256) acc_finish_kernel(const float *__restrict__ acc, void *__restrict__ out, int dtype, int64_t ldo,
                                                         int H, int64_t n4) {
  const int H4 = H / 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4 *>(acc)[i];
    const int64_t t = i / H4, c = 4 * (i - t * H4);
    store_from_f32(out, dtype, t * ldo + c, v.x);
    store_from_f32(out, dtype, t * ldo + c + 1, v.y);
    store_from_f32(out, dtype, t * ldo + c + 2, v.z);
    store_from_f32(out, dtype, t * ldo + c + 3, v.w);
  }
}

template <int NMAT, bool GATEUP, int CG, int FMT = 0>
int launch_tc_cg(TcParams p, int max_pairs, cudaStream_t st) {
  using S = Smem<NMAT, CG, FMT>;
  int dev = 0;
  KNJ_CUDA(cudaGetDevice(&dev));
  auto kern = q4k_grouped_tc_kernel<NMAT, GATEUP, CG, FMT>;
  static bool opted[64] = {false};
  if (dev >= 0 && dev < 64 && !opted[dev]) {
    KNJ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes));
    opted[dev] = true;
  }
  if (FMT == 0) {
    const uint64_t rows = (uint64_t)p.n_experts * p.N;
    int rc = make_row_tensor_map(&p.map0, p.W0, rows, (uint32_t)p.rowBytes, KNJ_Q4K_BYTES, 32);
    if (rc) return rc;
    if (GATEUP) {
      rc = make_row_tensor_map(&p.map1, p.W1, rows, (uint32_t)p.rowBytes, KNJ_Q4K_BYTES, 32);
      if (rc) return rc;
    }
  }
  // worst case number of token buckets: every expert has a ragged tail
  const long long buckets = (long long)max_pairs / kMaxTok + p.n_experts;
  const long long grid = buckets * p.m_tiles;
  KNJ_REQUIRE(grid > 0 && grid < (1ll << 31), "grouped GEMM: grid of %lld CTAs out of range", grid);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = S::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  KNJ_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  return launch_status("q4k_grouped_tc_kernel");
}

// pairs of CTAs whenever the row tiles of a bucket come in twos
template <int NMAT, bool GATEUP>
int launch_tc(const TcParams &p, int max_pairs, cudaStream_t st) {
  if (p.m_tiles % 2 == 0 && !g_tc_force_single) return launch_tc_cg<NMAT, GATEUP, 2>(p, max_pairs, st);
  return launch_tc_cg<NMAT, GATEUP, 1>(p, max_pairs, st);
}

}  // namespace

extern "C" {

#ifdef KNJ_TRACE
// Measurement hook (no reference counterpart): device buffer of 256 + 4 * cta_slots u64. SM-clock stamps of
// CTA 0: [4k..4k+3], k < 12: unpacker starts slab k, stage free, stage published, MMA sees the slab;
// [48..61] epilogue phases; [64+4k..], k < 12: loader reaches slab k, stage free, rows stored, published.
// From [256] on, per CTA b < cta_slots: global-timer ns at start, accumulator complete, end, and
// (SM id << 32 | tokens of its bucket).
void knj_trace_tc(void *dev_buf, int cta_slots) {
  g_tc_trace = static_cast<unsigned long long *>(dev_buf);
  g_tc_trace_ctas = dev_buf ? cta_slots : 0;
}
#endif

// 1 = run every bucket in the single-SM form (cta_group::1), the form buckets with an odd number of row tiles
// always take; 0 = CTA pairs wherever the tile count is even (default). Process-wide.
void knj_q4k_tc_single_sm(int on) { g_tc_force_single = on & 1; }

int knj_to_f16_launch(const void *x, int x_dtype, int64_t ldx, int rows, int K, void *out_f16, knj_stream_t s) {
  KNJ_REQUIRE(x && out_f16, "knj_to_f16: null pointer");
  KNJ_REQUIRE(x_dtype >= KNJ_DT_F32 && x_dtype <= KNJ_DT_F16 && K > 0, "knj_to_f16: bad dtype / K");
  if (rows <= 0) return KNJ_OK;
  const int64_t n = (int64_t)rows * K;
  if (x_dtype == KNJ_DT_BF16 && K % 8 == 0 && ldx % 8 == 0 && aligned16(x) && aligned16(out_f16)) {
    const int64_t n8 = n / 8, blocks8 = (n8 + 255) / 256, cap8 = (int64_t)sm_count() * 16;
    bf16_to_f16_kernel<<<(unsigned)(blocks8 < cap8 ? blocks8 : cap8), 256, 0, as_stream(s)>>>(
        static_cast<const uint4 *>(x), ldx / 8, K / 8, n8, static_cast<uint4 *>(out_f16));
    return launch_status("bf16_to_f16_kernel");
  }
  const int64_t blocks = (n + 255) / 256, cap = (int64_t)sm_count() * 16;
  to_f16_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, as_stream(s)>>>(x, x_dtype, ldx, K, n,
                                                                                  static_cast<__half *>(out_f16));
  return launch_status("to_f16_kernel");
}

int knj_q4k_gateup_tc_launch(const void *Xh, const uint8_t *Wg, const uint8_t *Wu, const int32_t *pair_idx,
                             const int32_t *pair_cnt, const int32_t *pair_tok, void *A_f16, int N, int K, int rowBytes,
                             int64_t idxStride, int n_experts, int top_k, int max_pairs, int *status, knj_stream_t s) {
  KNJ_REQUIRE(Xh && Wg && Wu && pair_idx && pair_cnt && A_f16, "knj_q4k_gateup_tc: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES, "knj_q4k_gateup_tc: rowBytes=%d does not match K=%d",
              rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % kRowsM == 0, "knj_q4k_gateup_tc: N=%d must be a multiple of 128", N);
  KNJ_REQUIRE(aligned16(Wg) && aligned16(Wu) && aligned16(Xh), "knj_q4k_gateup_tc: bases must be 16-byte aligned");
  KNJ_REQUIRE(n_experts >= 1 && n_experts <= 256 && (pair_tok || top_k >= 1) && max_pairs >= 0,
              "knj_q4k_gateup_tc: bad expert / pair counts");
  if (max_pairs == 0) return KNJ_OK;
  TcParams p{};
  p.X = static_cast<const __half *>(Xh); p.W0 = Wg; p.W1 = Wu; p.pair_idx = pair_idx; p.pair_cnt = pair_cnt;
  p.row_map = pair_tok; p.out = A_f16; p.N = N; p.K = K; p.rowBytes = rowBytes; p.row_div = top_k > 0 ? top_k : 1;
  p.n_experts = n_experts; p.m_tiles = N / kRowsM; p.idxStride = idxStride; p.out_scale = kActPrescale; p.status = status; KNJ_TC_SET_TRACE(p);
  return launch_tc<2, true>(p, max_pairs, as_stream(s));
}

int knj_q4k_down_tc_launch(const void *Ah, const uint8_t *Wd, const int32_t *pair_idx, const int32_t *pair_cnt,
                           const int32_t *pair_row, float *Y, int N, int K, int rowBytes, int64_t idxStride,
                           int n_experts, int max_pairs, int *status, knj_stream_t s) {
  KNJ_REQUIRE(Ah && Wd && pair_idx && pair_cnt && Y, "knj_q4k_down_tc: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES, "knj_q4k_down_tc: rowBytes=%d does not match K=%d",
              rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % kRowsM == 0, "knj_q4k_down_tc: N=%d must be a multiple of 128", N);
  KNJ_REQUIRE(aligned16(Wd) && aligned16(Ah), "knj_q4k_down_tc: bases must be 16-byte aligned");
  KNJ_REQUIRE(n_experts >= 1 && n_experts <= 256 && max_pairs >= 0, "knj_q4k_down_tc: bad expert / pair counts");
  if (max_pairs == 0) return KNJ_OK;
  TcParams p{};
  p.X = static_cast<const __half *>(Ah); p.W0 = Wd; p.W1 = nullptr; p.pair_idx = pair_idx; p.pair_cnt = pair_cnt;
  p.row_map = pair_row; p.out = Y; p.N = N; p.K = K; p.rowBytes = rowBytes; p.row_div = 1;
  p.n_experts = n_experts; p.idxStride = idxStride; p.out_scale = 1.0f / kActPrescale; p.status = status; KNJ_TC_SET_TRACE(p);
  if (N % (2 * kRowsM) == 0) {  // two row tiles per CTA share every gathered token tile
    p.m_tiles = N / (2 * kRowsM);
    return launch_tc<2, false>(p, max_pairs, as_stream(s));
  }
  p.m_tiles = N / kRowsM;
  return launch_tc<1, false>(p, max_pairs, as_stream(s));
}

// Grouped down GEMM over Q6_K weights (the mixed-format layers of Q4_K_M files): as knj_q4k_down_tc_launch with
// W6 [E][N][K/256][210]; K <= 1024 (the tile's rows are staged whole).
int knj_q6k_down_tc_launch(const void *Ah, const uint8_t *W6, const int32_t *pair_idx, const int32_t *pair_cnt,
                           const int32_t *pair_row, float *Y, int N, int K, int64_t idxStride, int n_experts, int max_pairs,
                           int *status, knj_stream_t s) {
  KNJ_REQUIRE(Ah && W6 && pair_idx && pair_cnt && Y, "knj_q6k_down_tc: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && K <= 256 * kQ6MaxSb, "knj_q6k_down_tc: K=%d must be a multiple of 256, at most %d", K, 256 * kQ6MaxSb);
  KNJ_REQUIRE(N > 0 && N % kRowsM == 0, "knj_q6k_down_tc: N=%d must be a multiple of 128", N);
  KNJ_REQUIRE(aligned16(W6) && aligned16(Ah), "knj_q6k_down_tc: bases must be 16-byte aligned");
  KNJ_REQUIRE(n_experts >= 1 && n_experts <= 256 && max_pairs >= 0, "knj_q6k_down_tc: bad expert / pair counts");
  if (max_pairs == 0) return KNJ_OK;
  TcParams p{};
  p.X = static_cast<const __half *>(Ah); p.W0 = W6; p.W1 = nullptr; p.pair_idx = pair_idx; p.pair_cnt = pair_cnt;
  p.row_map = pair_row; p.out = Y; p.N = N; p.K = K; p.rowBytes = K / 256 * KNJ_Q6K_BYTES; p.row_div = 1;
  p.n_experts = n_experts; p.idxStride = idxStride; p.out_scale = 1.0f / kActPrescale; p.status = status; KNJ_TC_SET_TRACE(p);
  p.m_tiles = N / kRowsM;
  if (p.m_tiles % 2 == 0 && !g_tc_force_single) return launch_tc_cg<1, false, 2, 1>(p, max_pairs, as_stream(s));
  return launch_tc_cg<1, false, 1, 1>(p, max_pairs, as_stream(s));
}

int knj_q4k_down_combine_tc_launch(const void *Ah, const uint8_t *Wd, const int32_t *pair_idx, const int32_t *pair_cnt,
                                   const int32_t *pair_row, const float *pair_w, int top_k, float *acc, int N, int K,
                                   int rowBytes, int64_t idxStride, int n_experts, int max_pairs, int *status, knj_stream_t s) {
  KNJ_REQUIRE(Ah && Wd && pair_idx && pair_cnt && pair_w && acc, "knj_q4k_down_combine_tc: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES, "knj_q4k_down_combine_tc: rowBytes=%d does not match K=%d",
              rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % kRowsM == 0, "knj_q4k_down_combine_tc: N=%d must be a multiple of 128", N);
  KNJ_REQUIRE(aligned16(Wd) && aligned16(Ah) && aligned16(acc), "knj_q4k_down_combine_tc: bases must be 16-byte aligned");
  KNJ_REQUIRE(n_experts >= 1 && n_experts <= 256 && max_pairs >= 0 && top_k >= 1, "knj_q4k_down_combine_tc: bad expert / pair counts");
  if (max_pairs == 0) return KNJ_OK;
  TcParams p{};
  p.X = static_cast<const __half *>(Ah); p.W0 = Wd; p.W1 = nullptr; p.pair_idx = pair_idx; p.pair_cnt = pair_cnt;
  p.row_map = pair_row; p.out = nullptr; p.N = N; p.K = K; p.rowBytes = rowBytes; p.row_div = 1;
  p.n_experts = n_experts; p.idxStride = idxStride; p.out_scale = 1.0f / kActPrescale; p.status = status; KNJ_TC_SET_TRACE(p);
  p.cmb_w = pair_w; p.cmb_acc = acc; p.cmb_div = top_k;
  if (N % (2 * kRowsM) == 0) {
    p.m_tiles = N / (2 * kRowsM);
    return launch_tc<2, false>(p, max_pairs, as_stream(s));
  }
  p.m_tiles = N / kRowsM;
  return launch_tc<1, false>(p, max_pairs, as_stream(s));
}

int knj_moe_acc_init_launch(const void *x, int x_dtype, int64_t ldx, int residual, int T, int H, float *acc, knj_stream_t s) {
  KNJ_REQUIRE(acc && (!residual || x) && T >= 0 && H > 0 && H % 4 == 0, "knj_moe_acc_init: bad arguments");
  if (T == 0) return KNJ_OK;
  const int64_t n4 = (int64_t)T * H / 4, blocks = (n4 + 255) / 256, cap = (int64_t)sm_count() * 16;
  acc_init_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, as_stream(s)>>>(x, x_dtype, ldx, residual, H, n4, acc);
  return launch_status("acc_init_kernel");
}

int knj_moe_acc_finish_launch(const float *acc, void *out, int out_dtype, int64_t ldo, int T, int H, knj_stream_t s) {
  KNJ_REQUIRE(acc && out && T >= 0 && H > 0 && H % 4 == 0, "knj_moe_acc_finish: bad arguments");
  if (T == 0) return KNJ_OK;
  const int64_t n4 = (int64_t)T * H / 4, blocks = (n4 + 255) / 256, cap = (int64_t)sm_count() * 16;
  acc_finish_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, as_stream(s)>>>(acc, out, out_dtype, ldo, H, n4);
  return launch_status("acc_finish_kernel");
}

}  // extern "C"
