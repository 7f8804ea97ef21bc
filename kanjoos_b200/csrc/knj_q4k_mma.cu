// knj_q4k_mma.cu -- decode-class expert projections: Q4_K weights streamed from
// HBM once, unpacked in registers and multiplied on the fp16 tensor cores as
// EXACT small integers, with the per-32 scale and min applied in f32.
//
// Why this shape. A Q4_K weight costs 0.5625 bytes; at HBM speed one SM must
// consume ~40 weights per clock, which a per-weight convert-and-fma loop on the
// CUDA cores cannot issue. So the 4-bit codes never become floats one by one:
//   * a code q placed in the low mantissa bits of an fp16 word IS the fp16
//     subnormal q * 2^-24 (or q * 2^-20 for a high nibble left in place), so
//     one AND per pair of weights builds a tensor-core A fragment;
//   * activations are split beforehand into a high and a low fp16 plane under a
//     per-vector power-of-two scale (together ~22 significant bits), so the
//     products and the f32 accumulation inside mma.sync are exact to f32 level;
//   * per 32-weight sub-block the integer-valued sum S = sum q*x comes out of
//     two m16n8k16 MMAs and is folded as  acc += (d*sc)*S - (dmin*m)*sum(x),
//     the factored form the reference's CPU decode uses
//     (src/loader/dequant.cpp:954-984 dot_q4_k).
// Weight rows reach shared memory through per-row bulk async copies
// (cp.async.bulk + mbarrier transaction bytes), one copy per lane, into rows
// padded so the fragment loads are bank-conflict free. No dequantised weight is
// ever written anywhere.
//
// Fragment bookkeeping. For one 32-byte code group (64 weights, sub-blocks 2G
// and 2G+1) lane (g = lane/4, t = lane%4) holds bytes 8t..8t+7 of rows g and
// g+8. Word s (s = 0,1) of those feeds MMA step s. Inside a word, bytes 0 and 2
// form the first k-pair and bytes 1 and 3 the second; the activation planes are
// stored with every aligned group of four k permuted to (0,2,1,3) so one
// 16-byte load yields the matching B fragments of both steps.
#include <type_traits>

#include "knj_common.cuh"
#include "knj_panel.cuh"
#include "knj_q4k.h"

using namespace knj;

namespace {

constexpr int kScalePitch = 18;  // floats per row of the scale table: 8 float2 + 1 pad pair

// ---------------------------------------------------------------------------
// activation prep: x -> (scale, hi plane, lo plane, per-32 sums), see knj_panel.cuh
// ---------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(128) act_prep_kernel(const void *__restrict__ x, int64_t ldx, int K,
                                                       uint8_t *__restrict__ panel) {
  __shared__ float red[16];
  const int v = blockIdx.x;
  grid_dep_wait();
  panel_prep_vector([&](int k) { return load_as_f32(x, DT, (int64_t)v * ldx + k); }, K,
                    panel + (size_t)v * panel_vec_bytes(K), red);
}

// ---------------------------------------------------------------------------
// the projection kernel
// ---------------------------------------------------------------------------
struct ProjParams {
  const uint8_t *W0;  // gate (dual) or the single matrix
  const uint8_t *W1;  // up (dual) or null
  const uint8_t *panel;
  const int32_t *pair_idx;
  const int32_t *pair_cnt;
  const int32_t *row_map;  // pair -> panel vector (null: pair / row_div)
  const int32_t *exp_list;
  const int32_t *n_active;
  float *out0;  // dual: G        single: Y
  float *out1;  // dual: U
  float *out2;  // dual: A = silu(G)*U
  int N, K, rowBytes, row_div, tiles_per_expert;
  int n_experts;  // length of exp_list / pair_cnt
  unsigned long long *trace;  // optional: [0..7] gate+up launch, [8..15] single-matrix launch
  int ks;         // warps that split the K range of one tile
  int tg;         // tiles per CTA (blockDim = 32 * tg * ks)
  int pitch;      // padded bytes per staged row part
  int tp_alloc;   // token slots per staged activation buffer
  int by_pass;    // 1: the work unit is (expert, tile group, token pass) instead of (expert, tile group)
  int resident;   // 1: whole panel vectors of a pass are staged at once (small batch); 0: one superblock chunk per step
  int64_t idxStride;
  int *status;    // optional: set to 1 when a bounded wait gave up
  CUtensorMap map0, map1;  // TMA descriptors of W0 / W1: box = this launch's row part x tile rows
  // optional fused weighted combine (single-matrix form only; cmb_out == null: off). The CTA that finishes a
  // column slice last (all active experts done) sums the slice for every token in ascending expert order.
  const int32_t *cmb_pair_exp;
  const float *cmb_pair_w;
  const void *cmb_resid;
  void *cmb_out;
  unsigned int *cmb_counter;  // one word per column slice, zero before the launch, left zero
  int64_t cmb_ld_resid, cmb_ldo;
  int cmb_resid_dtype, cmb_out_dtype, cmb_T, cmb_k;
};

struct ProjSmem {
  size_t weights, scales, bbuf, red, bars, total;
};
__host__ __device__ inline ProjSmem proj_smem(int warps, int pitch, int ks, int tp_alloc, int nt, int resident, int K) {
  ProjSmem m;
  m.weights = 0;
  m.scales = m.weights + (size_t)warps * 16 * pitch;
  m.bbuf = m.scales + (size_t)warps * 16 * kScalePitch * sizeof(float);
  m.red = m.bbuf + (resident ? (size_t)tp_alloc * panel_vec_bytes(K) : (size_t)2 * ks * tp_alloc * kChunkBytes);
  m.bars = m.red + (size_t)warps * 32 * 2 * nt * sizeof(float);
  m.total = m.bars + (size_t)(warps + 2) * 8 + 16;
  return m;
}

// One CTA = `tg` tiles of one expert x `ks` K-parts; warp w owns tile w / ks and
// the superblocks [part * nsb/ks, (part+1) * nsb/ks) with part = w % ks.
// DUAL: the m16 tile is 8 gate rows (fragment rows 0..7) + the 8 up rows of the
// same output indices (fragment rows 8..15), so silu(g)*u pairs up in-thread.
// Otherwise the tile is 16 consecutive rows of one matrix.
// All warps of the CTA walk the K steps in lockstep because they share the
// staged activation chunks (double buffered, one bulk copy per token and part).
template <bool DUAL, int NT>
__global__ void __launch_bounds__(512) q4k_proj_kernel(const __grid_constant__ ProjParams p) {
  constexpr int TP = 4 * NT;  // tokens per pass
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ks = p.ks, tile_slot = warp / ks, part = warp - tile_slot * ks;
  const int nsb = p.K / KNJ_QK_K, nsb_part = nsb / ks;
  const int part_bytes = nsb_part * KNJ_Q4K_BYTES;

  const ProjSmem lay = proj_smem(nwarp, p.pitch, ks, p.tp_alloc, NT, p.resident, p.K);
  uint8_t *wbase = smem + lay.weights + (size_t)warp * 16 * p.pitch;
  float *scales = reinterpret_cast<float *>(smem + lay.scales) + warp * 16 * kScalePitch;
  uint8_t *bbuf = smem + lay.bbuf;
  float *red = reinterpret_cast<float *>(smem + lay.red);
  uint64_t *wbar = reinterpret_cast<uint64_t *>(smem + lay.bars) + warp;
  uint64_t *bbar = reinterpret_cast<uint64_t *>(smem + lay.bars) + nwarp;
  volatile int *s_fail = reinterpret_cast<volatile int *>(bbar + 2);

  if (lane == 0) mbar_init(wbar, 1);
  if (threadIdx.x == 0) {
    mbar_init(&bbar[0], 1);
    mbar_init(&bbar[1], 1);
    *s_fail = 0;
  }
  mbar_init_fence();
  unsigned long long *tr = (p.trace && blockIdx.x == 0 && threadIdx.x == 0) ? p.trace + (DUAL ? 0 : 8) : nullptr;
  if (tr) tr[0] = global_timer_ns();
  grid_dep_wait();  // the plan, the prepared vectors (and for the down projection the activations) come from earlier launches
  __syncthreads();
  if (tr) tr[1] = global_timer_ns();
  uint32_t wphase = 0, bphase0 = 0, bphase1 = 0;
  bool ok = true;  // false: skip work and waits, but keep meeting the CTA barriers
  int staged_vec = -2;  // warp 0, lane i: the vector sitting in resident slot i

  // The plan is read with as few dependent round trips as possible (each costs most of a microsecond, and a
  // small batch has nothing else to hide them behind): the first item's expert is fetched together with the
  // number of active experts, later items' experts one item ahead, and an item's first pair ids together
  // with its pair count.
  const int groups = p.tiles_per_expert / p.tg;
  const int TPe = min(TP, p.tp_alloc);  // tokens per pass
  int e_next = 0;
  if (!p.by_pass && (int)blockIdx.x / groups < p.n_experts) e_next = p.exp_list[blockIdx.x / groups];
  const int n_act = p.n_active[0];
  int total = n_act * groups;
  const size_t vec_bytes = panel_vec_bytes(p.K);
  const int rows_per_tile = DUAL ? 8 : 16;
  const int first_lanes = min(TPe, (int)p.idxStride);

  // Batches whose experts can hold more tokens than one pass takes: the unit of work is one PASS of one tile
  // group, so that an expert with many tokens spreads over more CTAs instead of keeping a few of them busy
  // several times longer than the rest (its weight tile is then fetched once per pass, from L2 after the
  // first). Each CTA derives the same table: passes per active expert, exclusive prefix.
  __shared__ int s_ubase[257];
  __shared__ int s_uexp[256], s_ucnt[256];
  if (p.by_pass) {
    for (int a = threadIdx.x; a < 256; a += blockDim.x) {
      int c = 0, ex = -1;
      if (a < n_act) {
        ex = p.exp_list[a];
        c = p.pair_cnt[ex];
      }
      s_uexp[a] = ex;
      s_ucnt[a] = c;
      s_ubase[a] = (c + TPe - 1) / TPe;
    }
    __syncthreads();
    if (warp == 0) {
      int v[8], sum = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) { v[i] = s_ubase[lane * 8 + i]; sum += v[i]; }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      int base = incl - sum;
#pragma unroll
      for (int i = 0; i < 8; ++i) { s_ubase[lane * 8 + i] = base; base += v[i]; }
      if (lane == 31) s_ubase[256] = incl;
    }
    __syncthreads();
    total = s_ubase[256] * groups;
  }

  for (int it = blockIdx.x; it < total; it += gridDim.x) {
    int a, grp, e, cnt, tok_lo, tok_hi, pair_first = -1;
    if (p.by_pass) {
      const int pu = it / groups;
      grp = it - pu * groups;
      int lo = 0, hi = 255;  // the last a whose first pass is not beyond pu (inactive entries all hold the total)
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_ubase[mid] <= pu) lo = mid;
        else hi = mid - 1;
      }
      a = lo;
      e = s_uexp[a];
      cnt = s_ucnt[a];
      tok_lo = (pu - s_ubase[a]) * TPe;
      tok_hi = min(cnt, tok_lo + TPe);
    } else {
      a = it / groups;
      grp = it - a * groups;
      e = e_next;
      if (it + (int)gridDim.x < total) e_next = p.exp_list[(it + gridDim.x) / groups];
      pair_first = lane < first_lanes ? p.pair_idx[(size_t)e * p.idxStride + lane] : -1;
      cnt = p.pair_cnt[e];
      tok_lo = 0;
      tok_hi = cnt;
    }
    const int n0 = (grp * p.tg + tile_slot) * rows_per_tile;
    if (tr && it == (int)blockIdx.x) tr[2] = global_timer_ns() + (cnt & 0);

    // ---- this warp's part of the 16 weight rows: one TMA box per matrix (rows x part bytes), dense in
    // shared memory
    if (ok) {
      fence_proxy_async();
      if (lane == 0) {
        mbar_expect_tx(wbar, 16u * (uint32_t)part_bytes);
        const int xw = part * (part_bytes >> 2);
        if (DUAL) {
          tma_load_rows(wbase, &p.map0, xw, e * p.N + n0, wbar);
          tma_load_rows(wbase + 8 * part_bytes, &p.map1, xw, e * p.N + n0, wbar);
        } else {
          tma_load_rows(wbase, &p.map0, xw, e * p.N + n0, wbar);
        }
      }
    }
    bool w_ready = false;
    const uint8_t *rowA = wbase + (size_t)g * p.pitch;
    const uint8_t *rowB = wbase + (size_t)(g + 8) * p.pitch;

    for (int tok0 = tok_lo; tok0 < tok_hi; tok0 += TPe) {
      const int n_valid = min(TPe, cnt - tok0);
      // pair ids of this pass: lane i holds the pair of token tok0 + i
      int my_pair = -1, my_vec = -1;
      float my_inv = 0.f;  // the vector's inverse scale, needed only at the very end: fetched now
      if (lane < n_valid) {
        my_pair = (tok0 == 0 && !p.by_pass) ? pair_first : p.pair_idx[(size_t)e * p.idxStride + tok0 + lane];
        my_vec = p.row_map ? p.row_map[my_pair] : my_pair / p.row_div;
        my_inv = __ldg(reinterpret_cast<const float *>(p.panel + (size_t)my_vec * vec_bytes + (size_t)nsb * kChunkBytes));
      }
      // staged activation chunks: buffer b, part pp, token i
      auto stage_chunks = [&](int j) {
        if (warp == 0) {
          const int i = lane % p.tp_alloc, pp = lane / p.tp_alloc;
          const int vec = __shfl_sync(0xffffffffu, my_vec, i);
          uint64_t *bar = &bbar[j & 1];
          fence_proxy_async();
          if (lane == 0) mbar_expect_tx(bar, (uint32_t)(n_valid * ks) * kChunkBytes);
          __syncwarp();
          if (pp < ks && i < n_valid)
            bulk_g2s(bbuf + ((size_t)((j & 1) * ks + pp) * p.tp_alloc + i) * kChunkBytes,
                     p.panel + (size_t)vec * vec_bytes + (size_t)(pp * nsb_part + j) * kChunkBytes, kChunkBytes, bar);
        }
      };

      // resident mode: restage only when the vectors in shared memory are not the ones this pass needs.
      // The barrier doubles as "every warp is done with the activation buffers and the reduction scratch".
      bool restage = false;
      if (p.resident && warp == 0) restage = !__all_sync(0xffffffffu, lane >= n_valid || my_vec == staged_vec);
      const int any_restage = __syncthreads_or(restage ? 1 : 0);
      if (*s_fail) ok = false;
      bool have_b = false;
      if (p.resident) {
        have_b = any_restage == 0;
        if (ok && !have_b && warp == 0) {
          // one bulk copy per token: the whole prepared vector
          fence_proxy_async();
          if (lane == 0) mbar_expect_tx(&bbar[0], (uint32_t)n_valid * (uint32_t)(vec_bytes - 16));
          __syncwarp();
          if (lane < n_valid)
            bulk_g2s(bbuf + (size_t)lane * vec_bytes, p.panel + (size_t)my_vec * vec_bytes, (uint32_t)(vec_bytes - 16), &bbar[0]);
          staged_vec = lane < n_valid ? my_vec : -2;
        }
      } else if (ok) {
        stage_chunks(0);
      }

      float acc0[NT], acc1[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc0[nt] = acc1[nt] = 0.f;

      for (int j = 0; j < nsb_part; ++j) {
        if (!p.resident) {
          if (j + 1 < nsb_part) {
            __syncthreads();  // buffer (j+1)&1 was last read at step j-1
            if (ok) stage_chunks(j + 1);
          }
          if (ok) {
            uint32_t &bph = (j & 1) ? bphase1 : bphase0;
            if (!mbar_wait(&bbar[j & 1], bph, s_fail)) ok = false;
            bph ^= 1u;
          }
        } else if (ok && !have_b) {
          if (!mbar_wait(&bbar[0], bphase0, s_fail)) ok = false;
          bphase0 ^= 1u;
          have_b = true;
        }
        if (ok && !w_ready) {
          if (tr && it == (int)blockIdx.x) tr[3] = global_timer_ns();
          if (!mbar_wait(wbar, wphase, s_fail)) ok = false;
          wphase ^= 1u;
          w_ready = true;
          if (tr && it == (int)blockIdx.x) tr[4] = global_timer_ns();
        }
        if (!ok) continue;

        // ---- (d*sc, dmin*m) of 16 rows x 8 sub-blocks: lane -> row lane%16, sub-blocks 4*(lane/16)..+3
        __syncwarp();
        {
          const int r = lane & 15, hb = lane >> 4;
          const uint4 h = *reinterpret_cast<const uint4 *>(wbase + (size_t)r * p.pitch + (size_t)j * KNJ_Q4K_BYTES);
          const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
          const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
          const uint32_t sc4 = hb ? ((h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3f3f3f3fu);
          const uint32_t mn4 = hb ? (((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3f3f3f3fu);
          float2 *dst = reinterpret_cast<float2 *>(scales + r * kScalePitch) + 4 * hb;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float sc = (float)((sc4 >> (8 * i)) & 0xffu), mn = (float)((mn4 >> (8 * i)) & 0xffu);
            // even sub-blocks hold q*2^-24, odd ones q*2^-20
            dst[i] = make_float2(d * sc * ((i & 1) ? 1048576.0f : 16777216.0f), dmin * mn);
          }
        }
        __syncwarp();

        // chunk of (token slot, this step); unused slots alias the last staged one (their columns are discarded)
        const size_t slot_stride = p.resident ? vec_bytes : (size_t)kChunkBytes;
        const uint8_t *chunks = p.resident ? bbuf + (size_t)(part * nsb_part + j) * kChunkBytes
                                           : bbuf + (size_t)((j & 1) * ks + part) * p.tp_alloc * kChunkBytes;
        const int last_slot = p.tp_alloc - 1;
        float sx[NT][8];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const float4 *sp = reinterpret_cast<const float4 *>(chunks + (size_t)min(nt * 4 + t, last_slot) * slot_stride + kChunkSx);
          const float4 s0 = sp[0], s1 = sp[1];
          sx[nt][0] = s0.x; sx[nt][1] = s0.y; sx[nt][2] = s0.z; sx[nt][3] = s0.w;
          sx[nt][4] = s1.x; sx[nt][5] = s1.y; sx[nt][6] = s1.z; sx[nt][7] = s1.w;
        }
        const uint8_t *bfrag[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          bfrag[nt] = chunks + (size_t)min(nt * 4 + (g >> 1), last_slot) * slot_stride + (g & 1) * kChunkLo + 16 * t;

        // the inner loop, specialised on how many 4-token tiles of this pass hold tokens
        auto run = [&](auto nta_tag) {
          constexpr int NTA = decltype(nta_tag)::value;
#pragma unroll
          for (int G = 0; G < 4; ++G) {
            const size_t off = (size_t)j * KNJ_Q4K_BYTES + KNJ_Q4K_OFF_QS + 32 * G + 8 * t;
            const uint2 wa = *reinterpret_cast<const uint2 *>(rowA + off);
            const uint2 wb = *reinterpret_cast<const uint2 *>(rowB + off);
#pragma unroll
            for (int par = 0; par < 2; ++par) {
              const int sb = 2 * G + par;
              const uint32_t M = par ? 0x00f000f0u : 0x000f000fu;
              const float2 sa = *reinterpret_cast<const float2 *>(scales + g * kScalePitch + 2 * sb);
              const float2 sb2 = *reinterpret_cast<const float2 *>(scales + (g + 8) * kScalePitch + 2 * sb);
              const uint32_t a00 = wa.x & M, a01 = wb.x & M, a02 = (wa.x >> 8) & M, a03 = (wb.x >> 8) & M;
              const uint32_t a10 = wa.y & M, a11 = wb.y & M, a12 = (wa.y >> 8) & M, a13 = (wb.y >> 8) & M;
#pragma unroll
              for (int nt = 0; nt < NTA; ++nt) {
                const uint4 bf = *reinterpret_cast<const uint4 *>(bfrag[nt] + (64 * G + 32 * par) * 2);
                float c[4];
                mma_f16_16816_zero(c, a00, a01, a02, a03, bf.x, bf.y);
                mma_f16_16816(c, a10, a11, a12, a13, bf.z, bf.w);
                // columns 2t / 2t+1 are the high / low plane of the same token
                acc0[nt] = fmaf(sa.x, c[0] + c[1], acc0[nt]);
                acc0[nt] = fmaf(-sa.y, sx[nt][sb], acc0[nt]);
                acc1[nt] = fmaf(sb2.x, c[2] + c[3], acc1[nt]);
                acc1[nt] = fmaf(-sb2.y, sx[nt][sb], acc1[nt]);
              }
            }
          }
        };
        const int tiles = (n_valid + 3) >> 2;
        if (NT == 1 || tiles == 1) run(std::integral_constant<int, 1>{});
        else if (NT == 2 || tiles == 2) run(std::integral_constant<int, (NT >= 2 ? 2 : 1)>{});
        else if (tiles == 3) run(std::integral_constant<int, (NT >= 4 ? 3 : 1)>{});
        else run(std::integral_constant<int, NT>{});
      }

      if (tr && it == (int)blockIdx.x && tok0 == 0) tr[5] = global_timer_ns();
      // ---- combine the K parts (fixed order), undo the activation scale, store
      if (ks > 1) {
        float *mine = red + (size_t)(warp * 32 + lane) * 2 * NT;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { mine[2 * nt] = acc0[nt]; mine[2 * nt + 1] = acc1[nt]; }
        __syncthreads();
        if (part == 0) {
          for (int pp = 1; pp < ks; ++pp) {
            const float *other = red + (size_t)((warp + pp) * 32 + lane) * 2 * NT;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { acc0[nt] += other[2 * nt]; acc1[nt] += other[2 * nt + 1]; }
          }
        }
      }
      if (part == 0 && ok) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int pp = __shfl_sync(0xffffffffu, my_pair, nt * 4 + t);
          const float inv = __shfl_sync(0xffffffffu, my_inv, nt * 4 + t);
          if (pp < 0) continue;
          const float v0 = acc0[nt] * inv, v1 = acc1[nt] * inv;
          if (DUAL) {
            const size_t o = (size_t)pp * p.N + n0 + g;
            if (p.out0) p.out0[o] = v0;
            if (p.out1) p.out1[o] = v1;
            if (p.out2) p.out2[o] = (v0 / (1.0f + expf(-v0))) * v1;
          } else {
            p.out0[(size_t)pp * p.N + n0 + g] = v0;
            p.out0[(size_t)pp * p.N + n0 + g + 8] = v1;
          }
        }
      }
    }
    __syncwarp();

    if (!DUAL && p.cmb_out) {
      // ---- fused combine: did this CTA finish the column slice [grp * tg * 16, +tg * 16) as the last one?
      __shared__ int s_last;
      __shared__ unsigned char s_ord[64][8];
      __shared__ unsigned char s_cnt[64];
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned old = atomicAdd(&p.cmb_counter[grp], 1u);
        s_last = old == (unsigned)n_act - 1u;
        if (s_last) p.cmb_counter[grp] = 0u;  // ready for the next launch
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
        const int T = p.cmb_T, k = p.cmb_k;
        for (int t = threadIdx.x; t < T; t += blockDim.x) {  // the token's slots in ascending expert order
          int ex[8], ord[8];
          for (int sl = 0; sl < k; ++sl) { ex[sl] = p.cmb_pair_exp[t * k + sl]; ord[sl] = sl; }
          for (int a2 = 1; a2 < k; ++a2) {
            const int o = ord[a2], eo = ex[a2];
            int b2 = a2 - 1;
            while (b2 >= 0 && ex[b2] > eo) { ord[b2 + 1] = ord[b2]; ex[b2 + 1] = ex[b2]; --b2; }
            ord[b2 + 1] = o;
            ex[b2 + 1] = eo;
          }
          for (int sl = 0; sl < k; ++sl) s_ord[t][sl] = (unsigned char)ord[sl];
          s_cnt[t] = (unsigned char)k;
        }
        __syncthreads();
        const int width = p.tg * 16, c0 = grp * width;
        for (int idx = threadIdx.x; idx < T * width; idx += blockDim.x) {
          const int t = idx / width, c = c0 + idx - t * width;
          float acc = 0.f;
          for (int sl = 0; sl < k; ++sl) {
            const int pp = t * k + s_ord[t][sl];
            acc = __fadd_rn(acc, __fmul_rn(p.cmb_pair_w[pp], __ldcg(p.out0 + (size_t)pp * p.N + c)));
          }
          if (p.cmb_resid) acc = __fadd_rn(load_as_f32(p.cmb_resid, p.cmb_resid_dtype, (int64_t)t * p.cmb_ld_resid + c), acc);
          store_from_f32(p.cmb_out, p.cmb_out_dtype, (int64_t)t * p.cmb_ldo + c, acc);
        }
      }
      __syncthreads();
    }
  }
  if (tr) tr[6] = global_timer_ns();
  if (!ok && threadIdx.x == 0 && p.status) atomicExch(p.status, 1);
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

int pad_pitch(int rowBytes) {
  int pitch = rowBytes;
  while ((pitch % 128) != 32 && (pitch % 128) != 96) pitch += 16;
  return pitch;
}

// Experiment hook: 0 = choose automatically.
int g_force_ks = 0, g_force_tg = 0, g_force_nt = 0;
unsigned long long *g_proj_trace = nullptr;  // measurement hook: 16 global-timer stamps of CTA 0, warp 0

template <bool DUAL, int NT>
int launch_proj(ProjParams p, int n_experts_max, int max_tokens, cudaStream_t st) {
  const int nsb = p.K / KNJ_QK_K;
  const int TP = 4 * NT;
  p.n_experts = n_experts_max;
  p.trace = g_proj_trace;
  // small batches: split K over the warps of a CTA so every SM has many warps in flight,
  // and keep the whole prepared vectors of a pass resident in shared memory
  p.tp_alloc = max_tokens < TP ? (max_tokens < 1 ? 1 : max_tokens) : TP;
  p.resident = (size_t)p.tp_alloc * panel_vec_bytes(p.K) <= 40 * 1024 ? 1 : 0;
  p.by_pass = (max_tokens > TP && !p.cmb_out && n_experts_max <= 256) ? 1 : 0;
  // K-split: every part must fit one TMA box (at most 7 superblocks = 1008 bytes per row). Defaults measured
  // on B200 (48-layer resident stack, batch 1/8/64).
  auto fits = [&](int c) { return c >= 1 && nsb % c == 0 && nsb / c <= 7 && (p.resident || p.tp_alloc * c <= 32); };
  int ks = 0;
  for (int c = DUAL ? 2 : 1; c <= 16 && !ks; ++c)
    if (fits(c)) ks = c;
  if (!ks && fits(1)) ks = 1;
  if (g_force_ks > 0 && fits(g_force_ks)) ks = g_force_ks;
  KNJ_REQUIRE(ks >= 1, "q4k projection: rows of %d superblocks cannot be split into TMA boxes for this batch", nsb);
  int tg = (DUAL && max_tokens <= 4) ? 4 : 8;
  if (g_force_tg > 0) tg = g_force_tg;
  while (tg > 1 && (p.tiles_per_expert % tg != 0 || tg * ks > 16)) tg >>= 1;
  KNJ_REQUIRE(tg * ks <= 16, "q4k projection: K-split %d needs more than 16 warps", ks);
  p.ks = ks;
  p.tg = tg;
  p.pitch = nsb / ks * KNJ_Q4K_BYTES;  // dense TMA boxes
  {
    const uint64_t rows = (uint64_t)n_experts_max * p.N;
    int rc = make_row_tensor_map(&p.map0, p.W0, rows, (uint32_t)p.rowBytes, (uint32_t)p.pitch, DUAL ? 8 : 16);
    if (rc) return rc;
    if (DUAL) {
      rc = make_row_tensor_map(&p.map1, p.W1, rows, (uint32_t)p.rowBytes, (uint32_t)p.pitch, 8);
      if (rc) return rc;
    }
  }

  int dev = 0;
  KNJ_CUDA(cudaGetDevice(&dev));
  int smem_max = 0;
  KNJ_CUDA(cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  size_t smem = proj_smem(p.tg * ks, p.pitch, ks, p.tp_alloc, NT, p.resident, p.K).total;
  while (smem > (size_t)smem_max && p.tg > 1) {  // very long rows: fewer tiles per CTA
    p.tg >>= 1;
    smem = proj_smem(p.tg * ks, p.pitch, ks, p.tp_alloc, NT, p.resident, p.K).total;
  }
  KNJ_REQUIRE(smem <= (size_t)smem_max && p.tiles_per_expert % p.tg == 0,
              "q4k projection: rows of %d bytes do not fit the shared memory tile", p.rowBytes);
  const int threads = p.tg * ks * 32;
  auto kern = q4k_proj_kernel<DUAL, NT>;
  // opt in to the large dynamic shared memory once per device and instantiation
  // (kept out of later launches so they are plain stream work, capturable in a graph)
  static size_t opted[64] = {0};
  if (dev >= 0 && dev < 64 && opted[dev] < smem) {
    KNJ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    opted[dev] = smem;
  }
  int per_sm = (int)((size_t)(smem_max + 1024) / (smem + 1024));
  if (per_sm > 2048 / threads) per_sm = 2048 / threads;
  if (per_sm > 16) per_sm = 16;
  if (per_sm < 1) per_sm = 1;
  const long long max_items = (long long)n_experts_max * (p.tiles_per_expert / p.tg);
  long long grid = max_items;
  const long long cap = (long long)sm_count() * per_sm;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  KNJ_CUDA(launch_chain(kern, dim3((unsigned)grid), dim3(threads), smem, st, p));
  return launch_status("q4k_proj_kernel");
}

template <bool DUAL>
int launch_proj_nt(const ProjParams &p, int n_experts_max, int max_tokens, cudaStream_t st) {
  int nt = max_tokens <= 4 ? 1 : 2;  // 8 tokens per pass: experts of a decode batch rarely see more
  if (g_force_nt > 0) nt = g_force_nt;
  if (nt == 1) return launch_proj<DUAL, 1>(p, n_experts_max, max_tokens, st);
  if (nt == 2) return launch_proj<DUAL, 2>(p, n_experts_max, max_tokens, st);
  return launch_proj<DUAL, 4>(p, n_experts_max, max_tokens, st);
}

}  // namespace

extern "C" {

// Experiment hook for tuning runs: force the K-split and tiles-per-CTA of the
// decode projections (0 = automatic). Not part of the reference surface.
// Measurement hook (no reference counterpart): 16 uint64 that receive global-timer ns of CTA 0 / thread 0 of the
// decode projections -- [0] start, [1] predecessor complete, [2] plan read, [3] first wait for weights,
// [4] weights landed, [5] first pass computed, [6] end; +8 for the single-matrix launch. NULL = off.
void knj_q4k_proj_trace(void *dev_buf) { g_proj_trace = static_cast<unsigned long long *>(dev_buf); }

void knj_q4k_decode_tuning(int ks, int tg, int nt) {
  g_force_ks = ks;
  g_force_tg = tg;
  g_force_nt = nt;
}

size_t knj_panel_bytes(int n_vec, int K) { return (size_t)(n_vec > 0 ? n_vec : 0) * panel_vec_bytes(K); }

int knj_act_prep_launch(const void *x, int x_dtype, int64_t ldx, int n_vec, int K, void *panel, knj_stream_t s) {
  KNJ_REQUIRE(x && panel, "knj_act_prep: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0, "knj_act_prep: K=%d must be a multiple of 256", K);
  KNJ_REQUIRE(x_dtype >= KNJ_DT_F32 && x_dtype <= KNJ_DT_F16, "knj_act_prep: unknown dtype %d", x_dtype);
  KNJ_REQUIRE(aligned16(panel), "knj_act_prep: panel must be 16-byte aligned");
  if (n_vec <= 0) return KNJ_OK;
  uint8_t *pn = static_cast<uint8_t *>(panel);
  cudaError_t le;
  if (x_dtype == KNJ_DT_F32) le = launch_chain(act_prep_kernel<KNJ_DT_F32>, dim3(n_vec), dim3(128), 0, as_stream(s), x, ldx, K, pn);
  else if (x_dtype == KNJ_DT_BF16) le = launch_chain(act_prep_kernel<KNJ_DT_BF16>, dim3(n_vec), dim3(128), 0, as_stream(s), x, ldx, K, pn);
  else le = launch_chain(act_prep_kernel<KNJ_DT_F16>, dim3(n_vec), dim3(128), 0, as_stream(s), x, ldx, K, pn);
  KNJ_CUDA(le);
  return launch_status("act_prep_kernel");
}

int knj_q4k_gateup_launch(const void *Xpanel, const uint8_t *Wg, const uint8_t *Wu, const int32_t *pair_idx,
                          const int32_t *pair_cnt, const int32_t *pair_tok, const int32_t *exp_list,
                          const int32_t *n_active, float *G, float *U, float *A, int N, int K, int rowBytes,
                          int64_t idxStride, int n_experts, int top_k, int max_tokens, knj_stream_t s) {
  KNJ_REQUIRE(Xpanel && Wg && Wu && pair_idx && pair_cnt && exp_list && n_active, "knj_q4k_gateup: null pointer");
  KNJ_REQUIRE(G || U || A, "knj_q4k_gateup: no output requested");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES,
              "knj_q4k_gateup: rowBytes=%d does not match K=%d", rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % 8 == 0, "knj_q4k_gateup: N=%d must be a multiple of 8", N);
  KNJ_REQUIRE(aligned16(Wg) && aligned16(Wu) && aligned16(Xpanel), "knj_q4k_gateup: weights/panel must be 16-byte aligned");
  KNJ_REQUIRE(n_experts > 0 && (pair_tok || top_k > 0), "knj_q4k_gateup: bad expert / top_k count");
  ProjParams p{};
  p.W0 = Wg; p.W1 = Wu; p.panel = static_cast<const uint8_t *>(Xpanel);
  p.pair_idx = pair_idx; p.pair_cnt = pair_cnt; p.row_map = pair_tok; p.exp_list = exp_list; p.n_active = n_active;
  p.out0 = G; p.out1 = U; p.out2 = A;
  p.N = N; p.K = K; p.rowBytes = rowBytes; p.row_div = top_k > 0 ? top_k : 1;
  p.tiles_per_expert = N / 8; p.idxStride = idxStride; p.status = nullptr;
  return launch_proj_nt<true>(p, n_experts, max_tokens, as_stream(s));
}

int knj_q4k_proj_launch(const void *Apanel, const uint8_t *W, const int32_t *pair_idx, const int32_t *pair_cnt,
                        const int32_t *pair_row, const int32_t *exp_list, const int32_t *n_active, float *Y, int N,
                        int K, int rowBytes, int64_t idxStride, int n_experts, int max_tokens, knj_stream_t s) {
  KNJ_REQUIRE(Apanel && W && pair_idx && pair_cnt && exp_list && n_active && Y, "knj_q4k_proj: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES,
              "knj_q4k_proj: rowBytes=%d does not match K=%d", rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % 16 == 0, "knj_q4k_proj: N=%d must be a multiple of 16", N);
  KNJ_REQUIRE(aligned16(W) && aligned16(Apanel), "knj_q4k_proj: weights/panel must be 16-byte aligned");
  KNJ_REQUIRE(n_experts > 0, "knj_q4k_proj: bad expert count");
  ProjParams p{};
  p.W0 = W; p.W1 = nullptr; p.panel = static_cast<const uint8_t *>(Apanel);
  p.pair_idx = pair_idx; p.pair_cnt = pair_cnt; p.row_map = pair_row; p.exp_list = exp_list; p.n_active = n_active;
  p.out0 = Y; p.out1 = nullptr; p.out2 = nullptr;
  p.N = N; p.K = K; p.rowBytes = rowBytes; p.row_div = 1;
  p.tiles_per_expert = N / 16; p.idxStride = idxStride; p.status = nullptr;
  return launch_proj_nt<false>(p, n_experts, max_tokens, as_stream(s));
}

int knj_q4k_down_combine_launch(const void *Apanel, const uint8_t *W, const int32_t *pair_idx, const int32_t *pair_cnt,
                                const int32_t *exp_list, const int32_t *n_active, float *Y, int N, int K, int rowBytes,
                                int64_t idxStride, int n_experts, const int32_t *pair_exp, const float *pair_w,
                                const void *resid, int resid_dtype, int64_t ld_resid, void *out, int out_dtype,
                                int64_t ldo, int T, int k, uint32_t *counters, knj_stream_t s) {
  KNJ_REQUIRE(Apanel && W && pair_idx && pair_cnt && exp_list && n_active && Y && pair_exp && pair_w && out && counters,
              "knj_q4k_down_combine: null pointer");
  KNJ_REQUIRE(K > 0 && K % 256 == 0 && rowBytes == K / 256 * KNJ_Q4K_BYTES,
              "knj_q4k_down_combine: rowBytes=%d does not match K=%d", rowBytes, K);
  KNJ_REQUIRE(N > 0 && N % 16 == 0 && N / 16 <= 128 * 16, "knj_q4k_down_combine: N=%d must be a multiple of 16", N);
  KNJ_REQUIRE(aligned16(W) && aligned16(Apanel), "knj_q4k_down_combine: weights/panel must be 16-byte aligned");
  KNJ_REQUIRE(n_experts > 0 && T >= 1 && T <= 64 && k >= 1 && k <= 8, "knj_q4k_down_combine: at most 64 tokens, top-k of at most 8");
  KNJ_REQUIRE(out_dtype == KNJ_DT_F32 || out_dtype == KNJ_DT_BF16, "knj_q4k_down_combine: out must be f32 or bf16");
  KNJ_REQUIRE(!resid || (resid_dtype >= KNJ_DT_F32 && resid_dtype <= KNJ_DT_F16), "knj_q4k_down_combine: unknown residual dtype");
  ProjParams p{};
  p.W0 = W; p.W1 = nullptr; p.panel = static_cast<const uint8_t *>(Apanel);
  p.pair_idx = pair_idx; p.pair_cnt = pair_cnt; p.row_map = nullptr; p.exp_list = exp_list; p.n_active = n_active;
  p.out0 = Y; p.out1 = nullptr; p.out2 = nullptr;
  p.N = N; p.K = K; p.rowBytes = rowBytes; p.row_div = 1;
  p.tiles_per_expert = N / 16; p.idxStride = idxStride; p.status = nullptr;
  p.cmb_pair_exp = pair_exp; p.cmb_pair_w = pair_w; p.cmb_resid = resid; p.cmb_out = out; p.cmb_counter = counters;
  p.cmb_ld_resid = ld_resid; p.cmb_ldo = ldo; p.cmb_resid_dtype = resid_dtype; p.cmb_out_dtype = out_dtype;
  p.cmb_T = T; p.cmb_k = k;
  return launch_proj_nt<false>(p, n_experts, T, as_stream(s));
}

size_t knj_q4k_matmul_workspace_bytes(int m, int n_in) {
  if (m <= 0 || n_in <= 0) return 0;
  // panel + identity pair list + counts
  return ((knj_panel_bytes(m, n_in) + 255) & ~(size_t)255) + (((size_t)m * 4 + 255) & ~(size_t)255) + 256;
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
  void *panel = ws;
  ws += (knj_panel_bytes(m, n_in) + 255) & ~(size_t)255;
  int32_t *pair_idx = reinterpret_cast<int32_t *>(ws);
  ws += ((size_t)m * 4 + 255) & ~(size_t)255;
  int32_t *small = reinterpret_cast<int32_t *>(ws);  // [0] cnt, [1] exp_list, [2..3] n_active
  int rc = knj_act_prep_launch(x, x_dtype, ldx, m, n_in, panel, s);
  if (rc) return rc;
  iota_plan_kernel<<<(m + 255) / 256, 256, 0, as_stream(s)>>>(pair_idx, small + 0, small + 1, small + 2, m);
  rc = launch_status("iota_plan_kernel");
  if (rc) return rc;
  return knj_q4k_proj_launch(panel, W, pair_idx, small + 0, nullptr, small + 1, small + 2, y, n_out, n_in,
                             n_in / 256 * KNJ_Q4K_BYTES, m, 1, m, s);
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
