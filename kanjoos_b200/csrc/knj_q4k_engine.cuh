// knj_q4k_engine.cuh -- the tile engine of the decode-class expert projections:
// Q4_K weights streamed from HBM once through per-warp TMA rings, multiplied on
// the fp16 tensor cores as EXACT small integers, f32-accurate results.
//
// Arithmetic (the factored form of dot_q4_k, src/loader/dequant.cpp:954-984):
//   y[row][tok] = sum over superblocks of
//                 d * sum_sb sc_sb * sum_k q_k x_k  -  dmin * sum_sb m_sb * sum_k x_k
//   * a 4-bit code q left in place in an fp16 word IS the fp16 subnormal q * 2^-24
//     (q * 2^-20 for a high nibble), so one AND builds two A-fragment elements;
//   * one packed fp16 multiply folds the 6-bit sub-block scale in: q * sc < 1024
//     is still an exact fp16 subnormal, so a whole superblock accumulates inside
//     the tensor core and d is applied once per superblock and row in f32;
//   * activations are split into a high and a low fp16 plane under a power-of-two
//     scale per (token, superblock) -- together ~22 significant bits -- so the
//     products and the f32 accumulation of mma.sync are exact to f32 level; the
//     two planes of a token sit in adjacent MMA columns, so one m16n8k16 covers
//     four tokens and the planes are summed in-thread;
//   * the min term is one more MMA per superblock: A = the eight 6-bit m_sb,
//     B = the per-32 sums of the token's planes.
//
// Work split. A JOB is one expert with up to kJobTok of its tokens: four, i.e. one
// MMA column group (the code also carries the eight-token form, two column groups
// served by the same unpacked weights, which was measured slower); its activations
// are converted once per CTA into a PANEL in shared memory, laid out so that a
// warp's fragment loads are 128 contiguous bytes per quarter-warp. A warp owns a
// 16-row tile (8 gate + 8 up rows of the same output indices, or 16 rows of one
// matrix) for the whole K: it walks the superblocks, each arriving as one TMA box
// (16 rows x 144 bytes) in the warp's own ring, and keeps the running sums in
// registers. Warps never exchange anything; gate and up of an output meet in one
// thread, so SiLU*up is applied there.
//
// Fragment bookkeeping (m16n8k16, lane = 4 g + t). Lane t of a row owns code
// group t of the superblock: bytes 32t..32t+31 of qs = sub-block 2t in the low
// nibbles and sub-block 2t+1 in the high ones, so it needs only those two scales.
// Word i (bytes 4i..4i+3) feeds one MMA step per nibble kind: bytes 0 and 2 are
// the k pair (2t, 2t+1), bytes 1 and 3 the pair (2t+8, 2t+9). The activation
// planes keep every aligned group of four k in the order (0,2,1,3), so the B
// fragments of a step are 8 consecutive bytes. MMA column n = 2 * token + plane.
#pragma once
#include "knj_common.cuh"
#include "knj_q4k.h"

namespace knj {
namespace q4e {

constexpr int kTileRows = 16;
constexpr int kStageBytes = kTileRows * KNJ_Q4K_BYTES;  // 2304: one superblock column of a 16-row tile
constexpr int kJobTok = 4;                              // tokens of one job = one MMA column group (4 tokens x 2 planes = the MMA's n).
                                                        // 8 (two column groups for jobs of five and more tokens) is supported by the code
                                                        // below and measured slower: a two-group round costs twice a one-group round, so
                                                        // CTAs that drew such jobs ran 25 % above the mean of a phase
// Panel of one (token, superblock): eight 128-byte units u = 4 * (sub-block & 1) + (16-byte piece of the
// sub-block's plane); inside a unit, 16 bytes per (plane, t) at 16 * (4 * plane + t): the eight lanes of a
// quarter-warp (planes 0/1 of one token, t = 0..3) read one unit without bank conflicts. Then the per-32
// sums / 64 as fp16 pairs (sub-blocks 2t, 2t+1): high plane at 1024 + 4t, low plane at 1040 + 4t.
constexpr int kPanelBytes = 1088;

__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_h2(__half lo, __half hi) {
  return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

// x * sigmoid(x). The plain division would take its slow path whenever exp(-x) overflows; the fast one is
// within 2 ulp for divisors below 2^126 and returns 0 beyond, which is the limit value here.
__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.0f + expf(-x)); }

// Eight consecutive activations as f32 (16-byte aligned source).
__device__ __forceinline__ void load8_f32(const void *base, int dtype, int64_t elem, float (&v)[8]) {
  if (dtype == KNJ_DT_F32) {
    const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem);
    const float4 a = __ldcg(p), c = __ldcg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
  } else {
    const uint4 r = __ldcg(reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(base) + elem));
    const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (dtype == KNJ_DT_BF16) {
        v[2 * i] = __uint_as_float(u[i] << 16);
        v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2 *>(&u[i]);
        v[2 * i] = __low2float(h);
        v[2 * i + 1] = __high2float(h);
      }
    }
  }
}

// One warp converts the 256 values of one (token, superblock) -- lane l holds values 8l..8l+7 -- into the panel
// at `dst`; returns 1 / scale (the same in every lane).
__device__ __forceinline__ float panel_convert(const float (&v)[8], uint8_t *dst, int lane) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = warp_max(amax);
  // power-of-two scale that puts the largest magnitude in [2^13, 2^14)
  const int be = (int)(__float_as_uint(amax) >> 23);
  int e = 0;
  if (amax > 0.f && be != 0xff) e = max(-120, min(120, 140 - be));
  const float s = __uint_as_float((uint32_t)(127 + e) << 23);
  uint32_t hw[4], lw[4];
  float part = 0.f;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    __half hh[4], ll[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = v[4 * q + i] * s;
      hh[i] = __float2half_rn(f);
      const float hf = __half2float(hh[i]);
      ll[i] = __float2half_rn(f - hf);
      part += hf + __half2float(ll[i]);
    }
    hw[2 * q] = pack_h2(hh[0], hh[2]);
    hw[2 * q + 1] = pack_h2(hh[1], hh[3]);
    lw[2 * q] = pack_h2(ll[0], ll[2]);
    lw[2 * q + 1] = pack_h2(ll[1], ll[3]);
  }
  const int sb = lane >> 2, t = sb >> 1, u = 4 * (sb & 1) + (lane & 3);
  *reinterpret_cast<uint4 *>(dst + 128 * u + 16 * t) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
  *reinterpret_cast<uint4 *>(dst + 128 * u + 16 * (4 + t)) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
  part += __shfl_xor_sync(0xffffffffu, part, 1);
  part += __shfl_xor_sync(0xffffffffu, part, 2);              // the sub-block's sum, in its four lanes
  const float next = __shfl_down_sync(0xffffffffu, part, 4);  // the following sub-block's
  if ((lane & 7) == 0) {
    const float s0 = part * 0.015625f, s1 = next * 0.015625f;  // |sum| < 32 * 2^14: / 64 keeps it inside fp16
    const __half h0 = __float2half_rn(s0), h1 = __float2half_rn(s1);
    *reinterpret_cast<uint32_t *>(dst + 1024 + 4 * t) = pack_h2(h0, h1);
    *reinterpret_cast<uint32_t *>(dst + 1040 + 4 * t) =
        pack_h2(__float2half_rn(s0 - __half2float(h0)), __float2half_rn(s1 - __half2float(h1)));
  }
  return __uint_as_float((uint32_t)(127 - e) << 23);
}

// Weight row (0..7) that fragment row g of a lane stands for. A quarter-warp reads two rows at a time (g = 2j,
// 2j + 1), 64 bytes of each; they fall on disjoint shared-memory banks when the rows are 16 or 64 bytes apart
// modulo 128: adjacent rows for the 144-byte pitch, rows two apart for the 288-byte pitch.
__device__ __forceinline__ int tile_row(int g, int pitch) {
  return pitch == KNJ_Q4K_BYTES ? g : ((g & 4) | ((g & 1) << 1) | ((g >> 1) & 1));
}

// (sc[2t], sc[2t+1]) and (m[2t], m[2t+1]) of a superblock header as two bytes each (get_scale_min_k4,
// src/loader/dequant.cpp:64-77). sel16 picks halfword (t & 1) of a word, hi_var = (t >= 2).
__device__ __forceinline__ void header_pairs(const uint4 &hd, uint32_t sel16, bool hi_var, uint32_t &sc2, uint32_t &m2) {
  const uint32_t A = __byte_perm(hd.y, 0u, sel16), B = __byte_perm(hd.z, 0u, sel16), C = __byte_perm(hd.w, 0u, sel16);
  const uint32_t sc_lo = A & 0x3f3fu, m_lo = B & 0x3f3fu;
  const uint32_t sc_hi = (C & 0x0f0fu) | ((A >> 2) & 0x3030u);
  const uint32_t m_hi = ((C >> 4) & 0x0f0fu) | ((B >> 2) & 0x3030u);
  sc2 = hi_var ? sc_hi : sc_lo;
  m2 = hi_var ? m_hi : m_lo;
}

// One tile part: a superblock column of a 16-row tile (rows `pitch` bytes apart, the superblock at `stage` in
// each) times the panels of the job's tokens for that superblock (`pan`: token 0, token stride `tok_stride`
// bytes). NG = groups of four tokens (1 or 2). Lane (g, t) works on weight rows wrow and wrow + 8 of the tile
// (see tile_row) and receives, per group q, the superblock's contribution to (row wrow, token 4q + t) in
// rg[q] and to (row wrow + 8, token 4q + t) in rh[q], in the units of the token's scaled planes; the caller
// multiplies by 1 / scale. after_loads() runs once the weights are in registers (the stage may be refilled).
template <int NG, class AfterLoads>
__device__ __forceinline__ void tile_part(const uint8_t *stage, int pitch, int wrow, const uint8_t *pan, int tok_stride,
                                          int lane, float (&rg)[NG], float (&rh)[NG], AfterLoads after_loads) {
  const int g = lane >> 2, t = lane & 3;
  const uint8_t *wg_row = stage + wrow * pitch, *wh_row = stage + (wrow + 8) * pitch;
  const uint4 hg = *reinterpret_cast<const uint4 *>(wg_row), hh = *reinterpret_cast<const uint4 *>(wh_row);
  const uint4 wg0 = *reinterpret_cast<const uint4 *>(wg_row + KNJ_Q4K_OFF_QS + 32 * t);
  const uint4 wh0 = *reinterpret_cast<const uint4 *>(wh_row + KNJ_Q4K_OFF_QS + 32 * t);
  const uint4 wg1 = *reinterpret_cast<const uint4 *>(wg_row + KNJ_Q4K_OFF_QS + 32 * t + 16);
  const uint4 wh1 = *reinterpret_cast<const uint4 *>(wh_row + KNJ_Q4K_OFF_QS + 32 * t + 16);
  after_loads();
  const uint32_t wg[8] = {wg0.x, wg0.y, wg0.z, wg0.w, wg1.x, wg1.y, wg1.z, wg1.w};
  const uint32_t wh[8] = {wh0.x, wh0.y, wh0.z, wh0.w, wh1.x, wh1.y, wh1.z, wh1.w};
  // this lane's column in group q: token 4q + g / 2, plane g & 1
  const uint8_t *col = pan + (size_t)(g >> 1) * tok_stride;
  const uint8_t *bsrc = col + 16 * (4 * (g & 1) + t);
  const int grp_stride = 4 * tok_stride;

  const uint32_t sel16 = (t & 1) ? 0x4432u : 0x4410u;
  uint32_t scg, mg, sch, mh;
  header_pairs(hg, sel16, t >= 2, scg, mg);
  header_pairs(hh, sel16, t >= 2, sch, mh);
  // bytes -> fp16: 0x6400 | n is 1024 + n; the even scale is taken as is, the odd one (high nibbles, which
  // carry a factor 16) divided by 16 -- both exact
  const uint32_t k1024 = 0x64006400u, kSixteenth = 0x2c002c00u, kNeg64 = 0xd400d400u;
  const uint32_t sEg = sub_f16x2(__byte_perm(scg, 0x64646464u, 0x4040u), k1024);
  const uint32_t sOg = fma_f16x2(__byte_perm(scg, 0x64646464u, 0x4141u), kSixteenth, kNeg64);
  const uint32_t sEh = sub_f16x2(__byte_perm(sch, 0x64646464u, 0x4040u), k1024);
  const uint32_t sOh = fma_f16x2(__byte_perm(sch, 0x64646464u, 0x4141u), kSixteenth, kNeg64);
  const uint32_t mmg = sub_f16x2(__byte_perm(mg, 0x64646464u, 0x4140u), k1024);
  const uint32_t mmh = sub_f16x2(__byte_perm(mh, 0x64646464u, 0x4140u), k1024);

  // independent accumulator chains (the MMAs of one chain depend on each other): with one group, nibble kind
  // x step parity; with two groups, nibble kind x group
  constexpr int NC = NG == 1 ? 2 : 1;  // chains per (group, nibble kind)
  float cm[NG][4], ce[NG][NC][4], co[NG][NC][4];
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    const uint32_t sx = *reinterpret_cast<const uint32_t *>(col + q * grp_stride + 1024 + 16 * (g & 1) + 4 * t);
    mma_f16_16816_zero(cm[q], mmg, mmh, 0u, 0u, sx, 0u);
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
      for (int i = 0; i < 4; ++i) ce[q][c][i] = co[q][c][i] = 0.f;
  }
  // B fragments: one 16-byte load per (group, sub-block, step pair). One group: all eight loads go out first;
  // two groups: the loads of step pair j + 1 travel while pair j is multiplied.
  constexpr int NB = NG == 1 ? 4 : 2;  // step pairs held in registers
  uint4 be[NB][NG], bo[NB][NG];
#pragma unroll
  for (int j = 0; j < (NG == 1 ? 4 : 1); ++j)
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      be[j][q] = *reinterpret_cast<const uint4 *>(bsrc + q * grp_stride + 128 * j);
      bo[j][q] = *reinterpret_cast<const uint4 *>(bsrc + q * grp_stride + 128 * (4 + j));
    }
#pragma unroll
  for (int j = 0; j < 4; ++j) {  // steps 2j and 2j + 1
    const int cur = NG == 1 ? j : (j & 1);
    if (NG == 2 && j + 1 < 4) {
#pragma unroll
      for (int q = 0; q < NG; ++q) {
        be[(j + 1) & 1][q] = *reinterpret_cast<const uint4 *>(bsrc + q * grp_stride + 128 * (j + 1));
        bo[(j + 1) & 1][q] = *reinterpret_cast<const uint4 *>(bsrc + q * grp_stride + 128 * (4 + j + 1));
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int i = 2 * j + h;
      const uint32_t xg = wg[i], xh = wh[i], yg = xg >> 8, yh = xh >> 8;
      {
        const uint32_t a0 = mul_f16x2(xg & 0x000f000fu, sEg), a1 = mul_f16x2(xh & 0x000f000fu, sEh);
        const uint32_t a2 = mul_f16x2(yg & 0x000f000fu, sEg), a3 = mul_f16x2(yh & 0x000f000fu, sEh);
#pragma unroll
        for (int q = 0; q < NG; ++q)
          mma_f16_16816(ce[q][NC == 2 ? h : 0], a0, a1, a2, a3, h ? be[cur][q].z : be[cur][q].x, h ? be[cur][q].w : be[cur][q].y);
      }
      {
        const uint32_t a0 = mul_f16x2(xg & 0x00f000f0u, sOg), a1 = mul_f16x2(xh & 0x00f000f0u, sOh);
        const uint32_t a2 = mul_f16x2(yg & 0x00f000f0u, sOg), a3 = mul_f16x2(yh & 0x00f000f0u, sOh);
#pragma unroll
        for (int q = 0; q < NG; ++q)
          mma_f16_16816(co[q][NC == 2 ? h : 0], a0, a1, a2, a3, h ? bo[cur][q].z : bo[cur][q].x, h ? bo[cur][q].w : bo[cur][q].y);
      }
    }
  }
  // codes carried 2^-24, the sums 1/64; columns 2t and 2t+1 are the two planes of token t of the group
  const float dg = __half2float(__ushort_as_half((unsigned short)(hg.x & 0xffffu))) * 16777216.0f;
  const float ng = __half2float(__ushort_as_half((unsigned short)(hg.x >> 16))) * 64.0f;
  const float dh = __half2float(__ushort_as_half((unsigned short)(hh.x & 0xffffu))) * 16777216.0f;
  const float nh = __half2float(__ushort_as_half((unsigned short)(hh.x >> 16))) * 64.0f;
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    float sg = 0.f, sh = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      sg += (ce[q][c][0] + ce[q][c][1]) + (co[q][c][0] + co[q][c][1]);
      sh += (ce[q][c][2] + ce[q][c][3]) + (co[q][c][2] + co[q][c][3]);
    }
    rg[q] = dg * sg - ng * (cm[q][0] + cm[q][1]);
    rh[q] = dh * sh - nh * (cm[q][2] + cm[q][3]);
  }
}

// ---------------------------------------------------------------------------
// One projection phase of a CTA: its run [u0, u1) of the flat (job, tile) list.
// ---------------------------------------------------------------------------
constexpr int kWarps = 16;      // warps of a CTA that runs a phase
constexpr int kMaxStages = 4;   // TMA boxes in flight per warp, at most

struct JobTable {        // in shared memory, the same in every CTA
  int *jbase;            // [257] first job of active expert a; entries past the active ones hold the total
  int *uexp;             // [256] expert id of active expert a
};

struct PhaseShape {
  int N;                 // output rows per expert
  int nsb, sbs, stages;  // superblocks per row, per TMA box, boxes in flight per warp
  int tiles;             // tiles per expert: N / 8 (gate+up) or N / 16
};

struct PhaseSmem {       // per CTA
  uint8_t *ring;         // kWarps * stages * sbs * kStageBytes
  uint8_t *panels;       // kJobTok * nsb * kPanelBytes: the panels of the job in progress
  uint64_t *bars;        // kWarps * kMaxStages, initialised with count 1
  float *inv;            // [kJobTok][16]
  int *pair;             // [kJobTok]: output rows of the job's tokens, -1: no token in the slot
  float4 *red;           // [kWarps][32]: partial sums of the warps that share a tile (ksplit > 1 only)
  volatile int *fail;    // raised by the first wait that gives up
};

__host__ __device__ inline size_t phase_ring_bytes(int sbs, int stages) { return (size_t)kWarps * stages * sbs * kStageBytes; }
__host__ __device__ inline size_t phase_panel_bytes(int nsb) { return (size_t)kJobTok * nsb * kPanelBytes; }

// active expert of a job: the last a whose first job is not beyond it
__device__ __forceinline__ int job_locate(const int *jbase, int job) {
  int lo = 0, hi = 255;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (jbase[mid] <= job) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// Runs tiles [u0, u1) of the flat list, one job at a time. All kWarps * 32 threads of the CTA call it together
// (it contains CTA barriers). job_token(job, a, tk, pair, row) -> bool says whether token slot tk of the job
// exists and names its output row (pair) and its activation row; load_row(row, sb, lane, v) fetches values
// 256 sb + 8 lane .. + 7 of that activation row. out0/out1/out2 as for the launches: DUAL -> G, U, silu(G) * U;
// otherwise out0 = Y. Bit s of `parity` is the phase the warp's next wait on its barrier s expects (0 after
// initialisation); `ok` turns false when a wait gave up (the rest of the phase is then skipped, the CTA barriers
// are still met).
// ksplit (1, 2 or 4, a divisor of the boxes per tile): that many adjacent warps share a tile, each taking a
// contiguous part of its K range; their partial sums meet in sm.red (fixed order, two named barriers per tile).
// For runs with few tiles per warp, where a warp walking the whole K alone would be the critical path.
template <bool DUAL, class JobToken, class LoadRow>
__device__ __forceinline__ void run_phase(const PhaseShape &sh, const PhaseSmem &sm, const JobTable &jt, int u0, int u1,
                                          int ksplit, const CUtensorMap *map0, const CUtensorMap *map1, float *out0,
                                          float *out1, float *out2, long long wait_cycles, unsigned &parity, bool &ok,
                                          JobToken job_token, LoadRow load_row, int trace_mode = 0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int nsb = sh.nsb, S = sh.stages, sbs = sh.sbs, nbox = nsb / sbs, tiles = sh.tiles;
  const int stage_bytes = sbs * kStageBytes, pitch = sbs * KNJ_Q4K_BYTES;
  const int wrow = tile_row(g, pitch);
  const int rows_per_tile = DUAL ? 8 : 16;
  const int tok_stride = nsb * kPanelBytes;
  const int f = ksplit, nb = nbox / f;         // warps per tile, boxes per warp and tile
  const int part = warp % f, slot = warp / f;  // this warp's K part; its group's place among the CTA's tiles
  const int groups = kWarps / f;
  uint8_t *ring = sm.ring + (size_t)warp * S * stage_bytes;
  uint64_t *bars = sm.bars + warp * kMaxStages;
  if (u0 >= u1) return;
  const int jfirst = u0 / tiles, jlast = (u1 - 1) / tiles;
  for (int job = jfirst; job <= jlast; ++job) {
    const int a = job_locate(jt.jbase, job);
    // ---- this warp's tiles of the job: r0 + slot, r0 + slot + groups, ...; their first boxes leave before the
    // panels are built (weights do not depend on the activations)
    const int r0 = max(u0, job * tiles), r1 = min(u1, (job + 1) * tiles);
    const int n_mine = r0 + slot < r1 ? (r1 - r0 - slot + groups - 1) / groups : 0;
    const int n_items = n_mine * nb;
    const int row_base = jt.uexp[a] * sh.N + (r0 + slot - job * tiles) * rows_per_tile;
    // producer cursor: boxes are issued in the order they are consumed, so its stage is always the one the
    // consumer has just left once the ring is full. No divisions in the loops below: counters only.
    int p_left = n_items, p_stage = 0, p_bl = 0, p_row = row_base;
    auto issue_next = [&]() {
      if (lane == 0) {
        uint8_t *dst = ring + (size_t)p_stage * stage_bytes;
        const int x = (part * nb + p_bl) * (pitch / 4);
        fence_proxy_async();
        mbar_expect_tx(&bars[p_stage], (uint32_t)stage_bytes);
        tma_load_rows(dst, map0, x, p_row, &bars[p_stage]);
        if (DUAL) tma_load_rows(dst + 8 * pitch, map1, x, p_row, &bars[p_stage]);
      }
      if (++p_stage == S) p_stage = 0;
      if (++p_bl == nb) {
        p_bl = 0;
        p_row += groups * rows_per_tile;
      }
      --p_left;
    };
    if (ok && trace_mode != 2)
      for (int i = 0; i < S && p_left > 0; ++i) issue_next();

    __syncthreads();  // the previous job's tiles are done with the panels
    // ---- panels of the job: one warp per (token, superblock)
    for (int item = warp; item < kJobTok * nsb; item += kWarps) {
      const int sb = item % nsb, tk = item / nsb;
      int pair = -1, row = 0;
      const bool live = job_token(job, a, tk, pair, row);
      if (live) {
        float v[8];
        load_row(row, sb, lane, v);
        if (trace_mode != 3) {
          const float inv = panel_convert(v, sm.panels + (size_t)tk * tok_stride + (size_t)sb * kPanelBytes, lane);
          if (lane == 0) sm.inv[tk * 16 + sb] = inv;
        }
      }
      if (sb == 0 && lane == 0) sm.pair[tk] = live ? pair : -1;
    }
    __syncthreads();
    const bool two = kJobTok > 4 && sm.pair[kJobTok > 4 ? 4 : 0] >= 0;  // tokens fill the slots from 0 up: a fifth token means a second group

    int stage = 0;
    int n0 = (r0 + slot - job * tiles) * rows_per_tile;  // first output row of the tile in progress
    const int sb_first = part * nb * sbs;
    for (int ti = 0; ti < n_mine; ++ti, n0 += groups * rows_per_tile) {
      float rg[2] = {0.f, 0.f}, rh[2] = {0.f, 0.f};
      const uint8_t *pan = sm.panels + (size_t)sb_first * kPanelBytes;
      const float *inv = sm.inv + t * 16 + sb_first;
      for (int bl = 0; bl < nb; ++bl) {
        if (ok && trace_mode != 2) {
          if (!mbar_wait_for(&bars[stage], (parity >> stage) & 1u, wait_cycles, sm.fail)) ok = false;
          parity ^= 1u << stage;
        }
        if (ok) {
          if (trace_mode != 1) {
            const uint8_t *src = ring + (size_t)stage * stage_bytes;
            for (int k = 0; k < sbs; ++k, src += KNJ_Q4K_BYTES, pan += kPanelBytes, ++inv) {
              auto nothing = [] {};
              if (two) {
                float pg[2], ph[2];
                tile_part<2>(src, pitch, wrow, pan, tok_stride, lane, pg, ph, nothing);
                rg[0] = fmaf(pg[0], inv[0], rg[0]);
                rh[0] = fmaf(ph[0], inv[0], rh[0]);
                rg[1] = fmaf(pg[1], inv[64], rg[1]);
                rh[1] = fmaf(ph[1], inv[64], rh[1]);
              } else {
                float pg[1], ph[1];
                tile_part<1>(src, pitch, wrow, pan, tok_stride, lane, pg, ph, nothing);
                rg[0] = fmaf(pg[0], inv[0], rg[0]);
                rh[0] = fmaf(ph[0], inv[0], rh[0]);
              }
            }
          }
          __syncwarp();  // every lane is done with the box
          if (trace_mode != 2 && p_left > 0) issue_next();
        }
        if (++stage == S) stage = 0;
      }
      bool mine = true;
      if (f > 1) {  // the K parts of the tile meet; the group's first warp sums them in order and stores
        float4 *red = sm.red + (size_t)warp * 32 + lane;
        *red = make_float4(rg[0], rh[0], rg[1], rh[1]);
        asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * f) : "memory");
        mine = part == 0;
        if (mine) {
          for (int pp = 1; pp < f; ++pp) {
            const float4 o = red[(size_t)pp * 32];
            rg[0] += o.x; rh[0] += o.y; rg[1] += o.z; rh[1] += o.w;
          }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * f) : "memory");
      }
      if (mine && ok) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int pair = (q == 0 || two) ? sm.pair[4 * q + t] : -1;
          if (pair >= 0) {
            if (DUAL) {
              const size_t o = (size_t)pair * sh.N + n0 + wrow;
              if (out0) out0[o] = rg[q];
              if (out1) out1[o] = rh[q];
              if (out2) out2[o] = silu(rg[q]) * rh[q];
            } else {
              out0[(size_t)pair * sh.N + n0 + wrow] = rg[q];
              out0[(size_t)pair * sh.N + n0 + wrow + 8] = rh[q];
            }
          }
        }
      }
    }
  }
}

// How many warps should share a tile: more when the run has so few tiles per warp that one warp walking the
// whole K range would be the critical path. total_tiles over all CTAs, nbox boxes per tile.
__device__ __forceinline__ int choose_ksplit(long long total_tiles, int nbox, int n_ctas) {
  int f = 1;
  while (f < 4 && nbox % (2 * f) == 0 && total_tiles * f < 3ll * n_ctas * kWarps) f *= 2;
  return f;
}

// Jobs per active expert -> exclusive prefix in jbase[0..256] (jbase[a] holds the job count of active expert a on
// entry, 0 past the active ones). Called by warp 0 after a CTA barrier; a CTA barrier must follow.
__device__ __forceinline__ void job_prefix(int *jbase, int lane) {
  int v[8], sum = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) { v[i] = jbase[lane * 8 + i]; sum += v[i]; }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  int base = incl - sum;
#pragma unroll
  for (int i = 0; i < 8; ++i) { jbase[lane * 8 + i] = base; base += v[i]; }
  if (lane == 31) jbase[256] = incl;
}

}  // namespace q4e
}  // namespace knj
