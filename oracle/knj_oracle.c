/* knj_oracle.c -- CPU restatement of the reference's quantized MoE expert path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links or calls this
 * file; it exists so the CUDA kernels can be checked against the arithmetic the
 * reference performs on the CPU. Every function cites the reference source it
 * follows (paths are relative to the reference project root).
 *
 * Parity status: PINNED. The Q4_K decode, the fused Q4_K dot, the fp16
 * conversion and the W4-g128 GEMM are compared bit-for-bit against the
 * reference's own sources compiled unmodified (oracle/_ref, see ref_shim.cpp)
 * and against gguf-py; the committed golden vectors under tests/golden/ were
 * produced by that compiled reference.
 *
 * Build: see oracle/Makefile (plain C11 + pthreads for the column split).
 * Arithmetic note: compile WITHOUT -ffast-math and WITHOUT FMA contraction
 * (-ffp-contract=off); the reference's host build has neither.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define KNJ_OR_QK 256
#define KNJ_OR_Q4K_BYTES 144
#define KNJ_OR_Q6K_BYTES 210

/* ------------------------------------------------------------------------- */
/* column split over host threads                                            */
/* ------------------------------------------------------------------------- */
/* Output columns are independent, so how they are split over threads cannot
 * change a result; the reference splits them over its ThreadPool
 * (src/model/model.cpp:372-379). */
static int g_threads = 0; /* 0 = all online cores */

typedef void (*or_range_fn)(int j0, int j1, void* ctx);
typedef struct { or_range_fn fn; void* ctx; int j0, j1; } or_job;
static void* or_job_main(void* p) {
  or_job* j = (or_job*)p;
  j->fn(j->j0, j->j1, j->ctx);
  return NULL;
}

int knj_or_num_threads(void) {
  if (g_threads > 0) return g_threads;
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}
void knj_or_set_threads(int n) { g_threads = n > 0 ? n : 0; }

static void or_parallel_for(int n, int serial, or_range_fn fn, void* ctx) {
  int nt = knj_or_num_threads();
  if (nt > n) nt = n;
  if (serial || nt <= 1) { fn(0, n, ctx); return; }
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nt);
  or_job* jobs = (or_job*)malloc(sizeof(or_job) * (size_t)nt);
  const int per = (n + nt - 1) / nt;
  for (int t = 0; t < nt; ++t) {
    jobs[t].fn = fn; jobs[t].ctx = ctx;
    jobs[t].j0 = t * per < n ? t * per : n;
    jobs[t].j1 = (t + 1) * per < n ? (t + 1) * per : n;
    if (t > 0) pthread_create(&th[t], NULL, or_job_main, &jobs[t]);
  }
  or_job_main(&jobs[0]);
  for (int t = 1; t < nt; ++t) pthread_join(th[t], NULL);
  free(th); free(jobs);
}

/* ------------------------------------------------------------------------- */
/* scalar conversions                                                        */
/* ------------------------------------------------------------------------- */

/* fp16 bits -> f32, exact for every pattern.
 * Follows src/loader/dequant.cpp:1032-1055 (fp16_to_fp32) and its twins
 * kernels/knj_q4k.h:94-117, tests/host_oracle.h:39-61. */
float knj_or_fp16_to_fp32(uint16_t h) {
  uint32_t s = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = ((uint32_t)h >> 10) & 31u;
  uint32_t f = (uint32_t)h & 1023u;
  uint32_t out;
  if (e == 31u) {
    out = s | 0x7f800000u | (f << 13);
  } else if (e != 0u) {
    out = s | ((e + 112u) << 23) | (f << 13);
  } else if (f == 0u) {
    out = s;
  } else {
    /* subnormal half: value = f * 2^-24; shift the leading one up to bit 10 */
    int lz = 0;
    while (((f << lz) & 1024u) == 0u) ++lz;
    out = s | ((uint32_t)(113 - lz) << 23) | (((f << lz) & 1023u) << 13);
  }
  float r;
  memcpy(&r, &out, 4);
  return r;
}

/* bf16 bits -> f32. Follows src/loader/dequant.cpp:1068-1073. */
float knj_or_bf16_to_fp32(uint16_t b) {
  uint32_t w = (uint32_t)b << 16;
  float r;
  memcpy(&r, &w, 4);
  return r;
}

/* f32 -> bf16 bits, round to nearest even (NaN kept quiet). The reference has
 * no f32->bf16 routine; this matches torch / CUDA __float2bfloat16_rn and is
 * used only to build inputs. */
uint16_t knj_or_fp32_to_bf16(float v) {
  uint32_t w;
  memcpy(&w, &v, 4);
  if ((w & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((w >> 16) | 0x0040u);
  w += 0x7fffu + ((w >> 16) & 1u);
  return (uint16_t)(w >> 16);
}

static uint16_t rd_u16(const uint8_t* p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }

/* ------------------------------------------------------------------------- */
/* Q4_K                                                                      */
/* ------------------------------------------------------------------------- */

/* 6-bit (scale, min) of sub-block j in 0..7 out of the 12 packed bytes.
 * Follows src/loader/dequant.cpp:64-72 (get_scale_min_k4) ==
 * kernels/knj_q4k.h:135-144 (knj_q4k_scale_min). */
void knj_or_q4k_scale_min(const uint8_t* sc12, int j, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = sc12[j] & 63;
    *mn = sc12[j + 4] & 63;
  } else {
    *sc = (uint8_t)((sc12[j + 4] & 15) | ((sc12[j - 4] >> 6) << 4));
    *mn = (uint8_t)((sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4));
  }
}

/* One weight, superblock-local index r. Follows kernels/knj_q4k.h:147-167. */
float knj_or_q4k_weight(const uint8_t* blk, int r) {
  const float d = knj_or_fp16_to_fp32(rd_u16(blk));
  const float dmin = knj_or_fp16_to_fp32(rd_u16(blk + 2));
  const int j = r >> 5, l = r & 31;
  uint8_t sc, mn;
  knj_or_q4k_scale_min(blk + 4, j, &sc, &mn);
  const uint8_t byte = blk[16 + (j >> 1) * 32 + l];
  const float q = (float)((j & 1) ? (byte >> 4) : (byte & 15));
  const float d1 = d * (float)sc;
  const float m1 = dmin * (float)mn;
  return d1 * q - m1;
}

/* Sixteen consecutive weights from r0 (r0 % 16 == 0) with the (scale,min)
 * hoisted. Follows kernels/knj_q4k.h:215-231 (knj_q4k_span16). */
void knj_or_q4k_span16(const uint8_t* blk, int r0, float* out) {
  const float d = knj_or_fp16_to_fp32(rd_u16(blk));
  const float dmin = knj_or_fp16_to_fp32(rd_u16(blk + 2));
  const int j = r0 >> 5, l = r0 & 31;
  uint8_t sc, mn;
  knj_or_q4k_scale_min(blk + 4, j, &sc, &mn);
  const float d1 = d * (float)sc, m1 = dmin * (float)mn;
  const uint8_t* q = blk + 16 + (j >> 1) * 32 + l;
  for (int i = 0; i < 16; ++i) {
    const uint32_t v = (j & 1) ? (uint32_t)(q[i] >> 4) : (uint32_t)(q[i] & 15);
    out[i] = d1 * (float)v - m1;
  }
}

/* Row decode, n weights (n % 256 == 0). Follows
 * src/loader/dequant.cpp:102-125 (dequant_q4_k): 64 weights per 32 code bytes,
 * low nibbles first, then high nibbles. */
void knj_or_dequant_q4k(const uint8_t* src, float* dst, uint64_t n) {
  for (uint64_t b = 0; b < n / KNJ_OR_QK; ++b, src += KNJ_OR_Q4K_BYTES) {
    const float d = knj_or_fp16_to_fp32(rd_u16(src));
    const float dmin = knj_or_fp16_to_fp32(rd_u16(src + 2));
    const uint8_t* q = src + 16;
    for (int pair = 0; pair < 4; ++pair, q += 32, dst += 64) {
      uint8_t s0, m0, s1, m1;
      knj_or_q4k_scale_min(src + 4, 2 * pair, &s0, &m0);
      knj_or_q4k_scale_min(src + 4, 2 * pair + 1, &s1, &m1);
      const float da = d * (float)s0, ma = dmin * (float)m0;
      const float db = d * (float)s1, mb = dmin * (float)m1;
      for (int l = 0; l < 32; ++l) dst[l] = da * (float)(q[l] & 15) - ma;
      for (int l = 0; l < 32; ++l) dst[32 + l] = db * (float)(q[l] >> 4) - mb;
    }
  }
}

/* Fused decode-and-dot over nb superblocks. Follows
 * src/loader/dequant.cpp:954-984 (dot_q4_k): per 32-weight sub-block
 * d1*sum(q*x) - dm1*sum(x), f32 sequential sums, two sub-blocks interleaved. */
float knj_or_dot_q4k(const uint8_t* src, const float* x, uint64_t nb) {
  float acc = 0.0f;
  for (uint64_t b = 0; b < nb; ++b, src += KNJ_OR_Q4K_BYTES, x += KNJ_OR_QK) {
    const float d = knj_or_fp16_to_fp32(rd_u16(src));
    const float dmin = knj_or_fp16_to_fp32(rd_u16(src + 2));
    for (int pair = 0; pair < 4; ++pair) {
      uint8_t s0, m0, s1, m1;
      knj_or_q4k_scale_min(src + 4, 2 * pair, &s0, &m0);
      knj_or_q4k_scale_min(src + 4, 2 * pair + 1, &s1, &m1);
      const float da = d * (float)s0, ma = dmin * (float)m0;
      const float db = d * (float)s1, mb = dmin * (float)m1;
      const uint8_t* q = src + 16 + 32 * pair;
      const float* xa = x + 64 * pair;
      float qa = 0.0f, sa = 0.0f, qb = 0.0f, sb = 0.0f;
      for (int l = 0; l < 32; ++l) {
        qa += (float)(q[l] & 15) * xa[l];
        sa += xa[l];
        qb += (float)(q[l] >> 4) * xa[l + 32];
        sb += xa[l + 32];
      }
      acc += (da * qa - ma * sa) + (db * qb - mb * sb);
    }
  }
  return acc;
}

/* ------------------------------------------------------------------------- */
/* Q6_K (decoders for the mixed-format follow-up; same sources)              */
/* ------------------------------------------------------------------------- */

/* One weight. Follows kernels/knj_q4k.h:170-196 (knj_q6k_weight). */
float knj_or_q6k_weight(const uint8_t* blk, int r) {
  const float d = knj_or_fp16_to_fp32(rd_u16(blk + 208));
  const int8_t* sc = (const int8_t*)(blk + 192);
  const int half = r >> 7, t = r & 127, l = t & 31, qtr = t >> 5;
  const uint8_t* ql = blk + half * 64;
  const uint8_t* qh = blk + 128 + half * 32;
  const uint32_t lo = (qtr & 1) ? ql[l + 32] : ql[l];
  const uint32_t nib = (qtr < 2) ? (lo & 15u) : (lo >> 4);
  const uint32_t hi = (qh[l] >> (2 * qtr)) & 3u;
  const int q = (int)(nib | (hi << 4)) - 32;
  return d * (float)sc[half * 8 + (l >> 4) + 2 * qtr] * (float)q;
}

void knj_or_dequant_q6k(const uint8_t* src, float* dst, uint64_t n) {
  for (uint64_t b = 0; b < n / KNJ_OR_QK; ++b, src += KNJ_OR_Q6K_BYTES, dst += KNJ_OR_QK)
    for (int r = 0; r < KNJ_OR_QK; ++r) dst[r] = knj_or_q6k_weight(src, r);
}

/* ------------------------------------------------------------------------- */
/* matmul / rmsnorm / moe  (src/model/model.cpp)                             */
/* ------------------------------------------------------------------------- */

/* y[r][j] = sum_i W[j][i] * x[r][i] for a Q4_K weight whose rows (ggml
 * "columns", dims[0] fastest) are n_in long. Follows
 * src/model/model.cpp:326-380 (Model::matmul): m == 1 takes the fused dot,
 * m > 1 stages one 256-weight block and dots it per row, adding block partials
 * in block order. Output columns are independent, so the thread split cannot
 * change a result. */
typedef struct {
  const uint8_t* W; int n_in; const float* x; int m, ldx; float* y; int ldy;
} or_mm_q4k;
static void or_mm_q4k_cols(int j0, int j1, void* p) {
  const or_mm_q4k* a = (const or_mm_q4k*)p;
  const int nblk = a->n_in / KNJ_OR_QK;
  const uint64_t stride = (uint64_t)nblk * KNJ_OR_Q4K_BYTES;
  float buf[KNJ_OR_QK];
  for (int j = j0; j < j1; ++j) {
    const uint8_t* src = a->W + (uint64_t)j * stride;
    if (a->m == 1) {
      a->y[j] = knj_or_dot_q4k(src, a->x, (uint64_t)nblk);
      continue;
    }
    for (int r = 0; r < a->m; ++r) a->y[(size_t)r * a->ldy + j] = 0.0f;
    for (int b = 0; b < nblk; ++b) {
      knj_or_dequant_q4k(src + (uint64_t)b * KNJ_OR_Q4K_BYTES, buf, KNJ_OR_QK);
      for (int r = 0; r < a->m; ++r) {
        const float* xr = a->x + (size_t)r * a->ldx + (size_t)b * KNJ_OR_QK;
        float acc = 0.0f;
        for (int l = 0; l < KNJ_OR_QK; ++l) acc += buf[l] * xr[l];
        a->y[(size_t)r * a->ldy + j] += acc;
      }
    }
  }
}
void knj_or_matmul_q4k(const uint8_t* W, int n_in, int n_out, const float* x, int m, int ldx,
                       float* y, int ldy) {
  or_mm_q4k a = {W, n_in, x, m, ldx, y, ldy};
  const int serial = (uint64_t)n_in * (uint64_t)n_out * (uint64_t)m < (1u << 16);
  or_parallel_for(n_out, serial, or_mm_q4k_cols, &a);
}

/* Unquantized weight (block size 1): decode the column, then one sequential
 * f32 dot per row. Follows src/model/model.cpp:308-324 (matmul_plain).
 * wtype: 0 = f32, 1 = bf16, 2 = f16. */
typedef struct {
  const void* W; int wtype, n_in; const float* x; int m, ldx; float* y; int ldy;
} or_mm_plain;
static void or_mm_plain_cols(int j0, int j1, void* p) {
  const or_mm_plain* a = (const or_mm_plain*)p;
  float* col = (float*)malloc(sizeof(float) * (size_t)a->n_in);
  for (int j = j0; j < j1; ++j) {
    if (a->wtype == 0) {
      memcpy(col, (const float*)a->W + (size_t)j * a->n_in, sizeof(float) * (size_t)a->n_in);
    } else {
      const uint16_t* w16 = (const uint16_t*)a->W + (size_t)j * a->n_in;
      for (int i = 0; i < a->n_in; ++i)
        col[i] = (a->wtype == 1) ? knj_or_bf16_to_fp32(w16[i]) : knj_or_fp16_to_fp32(w16[i]);
    }
    for (int r = 0; r < a->m; ++r) {
      const float* xr = a->x + (size_t)r * a->ldx;
      float acc = 0.0f;
      for (int i = 0; i < a->n_in; ++i) acc += col[i] * xr[i];
      a->y[(size_t)r * a->ldy + j] = acc;
    }
  }
  free(col);
}
void knj_or_matmul_plain(const void* W, int wtype, int n_in, int n_out, const float* x, int m,
                         int ldx, float* y, int ldy) {
  or_mm_plain a = {W, wtype, n_in, x, m, ldx, y, ldy};
  const int serial = (uint64_t)n_in * (uint64_t)n_out * (uint64_t)m < (1u << 16);
  or_parallel_for(n_out, serial, or_mm_plain_cols, &a);
}

/* x * rsqrt(mean(x^2) + eps) * w per row. Follows
 * src/model/model.cpp:258-271 (rmsnorm_rows); w is already decoded to f32. */
void knj_or_rmsnorm_rows(const float* x, int m, int width, const float* w, float eps, float* out) {
  for (int r = 0; r < m; ++r) {
    const float* xr = x + (size_t)r * width;
    float* o = out + (size_t)r * width;
    float ss = 0.0f;
    for (int i = 0; i < width; ++i) ss += xr[i] * xr[i];
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = 0; i < width; ++i) o[i] = xr[i] * scale * w[i];
  }
}

/* silu. Follows src/model/model.cpp:47. */
static float or_silu(float v) { return v / (1.0f + expf(-v)); }

/* g[i] = silu(g[i]) * u[i], the activation stage of the MoE branch.
 * Follows src/model/model.cpp:487-492. */
void knj_or_silu_mul(float* g, const float* u, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) g[i] = or_silu(g[i]) * u[i];
}

/* Router only: logits -> softmax over E -> K-pass arg-max (strict '>' so ties
 * go to the lowest expert id) -> renormalise. Follows
 * src/model/model.cpp:419-460. Outputs per token: chosen[K] in selection order
 * (descending probability) and weight[K]; logits may be NULL. */
void knj_or_route(const void* Wr, int wr_type, const float* hx, int m, int H, int E, int K,
                  float* logits_out, int32_t* chosen_out, float* weight_out) {
  float* rlog = (float*)malloc(sizeof(float) * (size_t)m * E);
  float* probs = (float*)malloc(sizeof(float) * (size_t)E);
  knj_or_matmul_plain(Wr, wr_type, H, E, hx, m, H, rlog, E);
  for (int t = 0; t < m; ++t) {
    const float* lg = rlog + (size_t)t * E;
    int32_t* chosen = chosen_out + (size_t)t * K;
    float mx = lg[0];
    for (int e = 1; e < E; ++e) mx = lg[e] > mx ? lg[e] : mx;
    float sum = 0.0f;
    for (int e = 0; e < E; ++e) {
      probs[e] = expf(lg[e] - mx);
      sum += probs[e];
    }
    for (int e = 0; e < E; ++e) probs[e] /= sum;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      for (int e = 0; e < E; ++e) {
        int taken = 0;
        for (int q = 0; q < k; ++q) taken |= (chosen[q] == e);
        if (taken) continue;
        if (best < 0 || probs[e] > probs[best]) best = e;
      }
      chosen[k] = best;
    }
    float keep = 0.0f;
    for (int k = 0; k < K; ++k) keep += probs[chosen[k]];
    const float inv = keep > 0.0f ? 1.0f / keep : 0.0f;
    for (int k = 0; k < K; ++k) weight_out[(size_t)t * K + k] = probs[chosen[k]] * inv;
  }
  if (logits_out) memcpy(logits_out, rlog, sizeof(float) * (size_t)m * E);
  free(rlog);
  free(probs);
}

/* The whole MoE branch for m rows. Follows src/model/model.cpp:399-510
 * (Model::moe): route, zero the output, then for each expert in ASCENDING id
 * gather its rows, gate, up, silu(g)*u, down, and out[row] += w * y.
 * Weights: Wg, Wu = Q4_K [E][F][H/256][144]; Wd = Q4_K [E][H][F/256][144].
 * Optional taps (may be NULL): chosen/weight [m][K]. */
void knj_or_moe(const void* Wr, int wr_type, const uint8_t* Wg, const uint8_t* Wu,
                const uint8_t* Wd, const float* hx, int m, int H, int E, int K, int F, float* out,
                int32_t* chosen_tap, float* weight_tap) {
  int32_t* chosen = (int32_t*)malloc(sizeof(int32_t) * (size_t)m * K);
  float* weight = (float*)malloc(sizeof(float) * (size_t)m * K);
  knj_or_route(Wr, wr_type, hx, m, H, E, K, NULL, chosen, weight);

  int32_t* rows = (int32_t*)malloc(sizeof(int32_t) * (size_t)m);
  float* rw = (float*)malloc(sizeof(float) * (size_t)m);
  float* gat = (float*)malloc(sizeof(float) * (size_t)m * H);
  float* yg = (float*)malloc(sizeof(float) * (size_t)m * F);
  float* yu = (float*)malloc(sizeof(float) * (size_t)m * F);
  float* yd = (float*)malloc(sizeof(float) * (size_t)m * H);
  const uint64_t gu_slab = (uint64_t)F * (uint64_t)(H / KNJ_OR_QK) * KNJ_OR_Q4K_BYTES;
  const uint64_t dn_slab = (uint64_t)H * (uint64_t)(F / KNJ_OR_QK) * KNJ_OR_Q4K_BYTES;

  memset(out, 0, sizeof(float) * (size_t)m * H);
  for (int e = 0; e < E; ++e) {
    int cnt = 0;
    for (int t = 0; t < m; ++t)
      for (int k = 0; k < K; ++k)
        if (chosen[(size_t)t * K + k] == e) {
          rows[cnt] = t;
          rw[cnt] = weight[(size_t)t * K + k];
          ++cnt;
        }
    if (cnt == 0) continue;
    for (int r = 0; r < cnt; ++r)
      memcpy(gat + (size_t)r * H, hx + (size_t)rows[r] * H, sizeof(float) * (size_t)H);
    knj_or_matmul_q4k(Wg + (uint64_t)e * gu_slab, H, F, gat, cnt, H, yg, F);
    knj_or_matmul_q4k(Wu + (uint64_t)e * gu_slab, H, F, gat, cnt, H, yu, F);
    for (size_t i = 0, n = (size_t)cnt * F; i < n; ++i) yg[i] = or_silu(yg[i]) * yu[i];
    knj_or_matmul_q4k(Wd + (uint64_t)e * dn_slab, F, H, yg, cnt, F, yd, H);
    for (int r = 0; r < cnt; ++r) {
      float* dst = out + (size_t)rows[r] * H;
      const float* src = yd + (size_t)r * H;
      const float wt = rw[r];
      for (int i = 0; i < H; ++i) dst[i] += wt * src[i];
    }
  }
  if (chosen_tap) memcpy(chosen_tap, chosen, sizeof(int32_t) * (size_t)m * K);
  if (weight_tap) memcpy(weight_tap, weight, sizeof(float) * (size_t)m * K);
  free(chosen); free(weight); free(rows); free(rw); free(gat); free(yg); free(yu); free(yd);
}

/* Routing plan of the device benches: double-precision logits from an f32
 * router weight [E][H], softmax, exact descending order with ascending-id
 * tie-break, renormalised weight per pair p = t*K + s, and the permutation
 * tables pairIdx[E][T] (-1 padded), pairCnt[E]. Follows
 * tools/bench/q4k_stream_ffn.hip:957-1001 (build_plan) ==
 * tools/bench/q4k_moe_ffn.hip:501-550. Returns maxCnt. */
int knj_or_build_plan(const float* x, const float* Wr32, int T, int H, int E, int K, float* rw,
                      int32_t* pairTok, int32_t* pairExp, int32_t* pairIdx, int32_t* pairCnt) {
  float* lg = (float*)malloc(sizeof(float) * (size_t)E);
  int* order = (int*)malloc(sizeof(int) * (size_t)E);
  for (size_t i = 0; i < (size_t)E * T; ++i) pairIdx[i] = -1;
  for (int e = 0; e < E; ++e) pairCnt[e] = 0;
  for (int t = 0; t < T; ++t) {
    for (int e = 0; e < E; ++e) {
      double acc = 0.0;
      for (int h = 0; h < H; ++h) acc += (double)x[(size_t)t * H + h] * (double)Wr32[(size_t)e * H + h];
      lg[e] = (float)acc;
    }
    double mx = -1e300, sum = 0.0;
    for (int e = 0; e < E; ++e) mx = (double)lg[e] > mx ? (double)lg[e] : mx;
    for (int e = 0; e < E; ++e) sum += exp((double)lg[e] - mx);
    for (int e = 0; e < E; ++e) order[e] = e;
    for (int a = 0; a < E; ++a)
      for (int b = a + 1; b < E; ++b)
        if (lg[order[b]] > lg[order[a]] || (lg[order[b]] == lg[order[a]] && order[b] < order[a])) {
          int tmp = order[a]; order[a] = order[b]; order[b] = tmp;
        }
    double ksum = 0.0;
    for (int s = 0; s < K; ++s) ksum += exp((double)lg[order[s]] - mx) / sum;
    for (int s = 0; s < K; ++s) {
      const int e = order[s], p = t * K + s;
      pairTok[p] = t;
      pairExp[p] = e;
      rw[p] = (float)((exp((double)lg[e] - mx) / sum) / (ksum > 0 ? ksum : 1.0));
      pairIdx[(size_t)e * T + pairCnt[e]++] = p;
    }
  }
  int mc = 0;
  for (int e = 0; e < E; ++e) mc = pairCnt[e] > mc ? pairCnt[e] : mc;
  free(lg); free(order);
  return mc;
}

/* ------------------------------------------------------------------------- */
/* W4-g128 path (tests/host_oracle.h, kernels/knj_pack.h)                    */
/* ------------------------------------------------------------------------- */

/* Dequantise-then-multiply in double over natural-order int8 activations.
 * Follows tests/host_oracle.h:77-104 (gemm_w4_reference); group = 128 weights,
 * 64 payload bytes + fp16 scale + zp + pad = 68 bytes, code bias 8. */
void knj_or_gemm_w4_reference(const uint8_t* Bq, const int8_t* Act, float* C, int M, int N, int K) {
  const int groups = K / 128;
  for (int m = 0; m < M; ++m) {
    const int8_t* a = Act + (size_t)m * K;
    for (int n = 0; n < N; ++n) {
      double acc = 0.0;
      for (int g = 0; g < groups; ++g) {
        const uint8_t* grp = Bq + ((size_t)n * groups + g) * 68;
        const float scale = knj_or_fp16_to_fp32(rd_u16(grp + 64));
        double inner = 0.0;
        for (int j = 0; j < 64; ++j) {
          inner += (double)((int)(grp[j] & 15) - 8) * (double)a[g * 128 + 2 * j];
          inner += (double)((int)(grp[j] >> 4) - 8) * (double)a[g * 128 + 2 * j + 1];
        }
        acc += (double)scale * inner;
      }
      C[(size_t)m * N + n] = (float)acc;
    }
  }
}

/* Natural-order int8 -> [M][K/8][2] u32 (even offsets, odd offsets). Follows
 * tests/host_oracle.h:110-134 == kernels/knj_pack.h:208-222. */
void knj_or_deinterleave_activations(const int8_t* Act, uint32_t* Out, int M, int K) {
  for (int m = 0; m < M; ++m)
    for (int j = 0; j < K / 8; ++j) {
      uint32_t ev = 0, od = 0;
      for (int t = 0; t < 4; ++t) {
        ev |= (uint32_t)(uint8_t)Act[(size_t)m * K + j * 8 + 2 * t] << (8 * t);
        od |= (uint32_t)(uint8_t)Act[(size_t)m * K + j * 8 + 2 * t + 1] << (8 * t);
      }
      Out[((size_t)m * (K / 8) + j) * 2 + 0] = ev;
      Out[((size_t)m * (K / 8) + j) * 2 + 1] = od;
    }
}

/* Per (m, group) activation sums: what kernels/knj_kernels.hip:232-260
 * (knj_build_asum) must produce, computed the plain way. */
void knj_or_build_asum(const int8_t* Act, int32_t* Asum, int M, int K) {
  const int groups = K / 128;
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < groups; ++g) {
      int32_t s = 0;
      for (int k = 0; k < 128; ++k) s += Act[(size_t)m * K + g * 128 + k];
      Asum[(size_t)m * groups + g] = s;
    }
}

/* The device-side formula in integers, for an exact cross-check of the CUDA
 * kernel: C = sum_g scale_g * ((float)raw_g - (float)(8*Asum_g)), f32
 * accumulate in group order. Follows kernels/knj_kernels.hip:176-218. */
void knj_or_gemm_w4_i8_mirror(const uint8_t* Bq, const int8_t* Act, float* C, int M, int N, int K) {
  const int groups = K / 128;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = 0.0f;
      for (int g = 0; g < groups; ++g) {
        const uint8_t* grp = Bq + ((size_t)n * groups + g) * 68;
        const float scale = knj_or_fp16_to_fp32(rd_u16(grp + 64));
        int32_t raw = 0, asum = 0;
        for (int j = 0; j < 64; ++j) {
          const int a0 = Act[(size_t)m * K + g * 128 + 2 * j];
          const int a1 = Act[(size_t)m * K + g * 128 + 2 * j + 1];
          raw += (int)(grp[j] & 15) * a0 + (int)(grp[j] >> 4) * a1;
          asum += a0 + a1;
        }
        acc += scale * ((float)raw - (float)(8 * asum));
      }
      C[(size_t)m * N + n] = acc;
    }
}

/* f32 -> fp16 bits by truncation toward zero, no subnormals. Follows
 * src/loader/dequant.cpp:1057-1066 (fp32_to_fp16); exact for the small
 * integers the W4 known-answer test feeds it. */
uint16_t knj_or_fp32_to_fp16_trunc(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t e = (int32_t)((x >> 23) & 255u) - 127 + 15;
  if (e <= 0) return (uint16_t)sign;
  if (e >= 31) return (uint16_t)(sign | 0x7c00u);
  return (uint16_t)(sign | ((uint32_t)e << 10) | ((x & 0x7fffffu) >> 13));
}

/* The seeded W4 known-answer problem: xorshift32 from `seed`, scales 6..10,
 * codes 0..15 (low nibble drawn first), zero point byte 8, pad 0, then
 * activations uniform in [-24, 24]. Follows tests/test_gemm_w4.hip:107-116
 * (generator) and :188-226 (draw order). */
static uint32_t xs32(uint32_t* s) {
  uint32_t x = *s;
  x ^= x << 13; x ^= x >> 17; x ^= x << 5;
  *s = x;
  return x;
}
void knj_or_w4_kat_problem(uint32_t seed, int M, int N, int K, uint8_t* Bq, int8_t* Act) {
  uint32_t s = seed ? seed : 1u;
  const int groups = K / 128;
  for (int n = 0; n < N; ++n)
    for (int g = 0; g < groups; ++g) {
      uint8_t* grp = Bq + ((size_t)n * groups + g) * 68;
      const int q = 6 + (int)(xs32(&s) % 5u);
      const uint16_t hb = knj_or_fp32_to_fp16_trunc((float)q);
      grp[64] = (uint8_t)(hb & 255u);
      grp[65] = (uint8_t)(hb >> 8);
      grp[66] = 8;
      grp[67] = 0;
      for (int j = 0; j < 64; ++j) {
        const uint8_t c0 = (uint8_t)(xs32(&s) & 15u);
        const uint8_t c1 = (uint8_t)(xs32(&s) & 15u);
        grp[j] = (uint8_t)((c1 << 4) | c0);
      }
    }
  for (size_t i = 0; i < (size_t)M * K; ++i) Act[i] = (int8_t)(-24 + (int32_t)(xs32(&s) % 49u));
}

/* Error metric the reference reports everywhere. Follows
 * tests/host_oracle.h:143-171 (ErrorStats / compare): relative RMSE over the
 * elements whose expected value is nonzero, max-abs + its index, RMS of the
 * expected output, count of nonzero produced outputs.
 * out[0..5] = rel_rmse, max_abs, out_rms, max_idx, nonzero, total. */
void knj_or_compare(const float* got, const float* want, int64_t total, double* out) {
  double se = 0.0, sw = 0.0, max_abs = 0.0;
  int64_t max_idx = -1, nonzero = 0;
  for (int64_t i = 0; i < total; ++i) {
    if (want[i] != 0.0f) {
      const double d = (double)(got[i] - want[i]);
      se += d * d;
      sw += (double)want[i] * (double)want[i];
    }
    const double a = fabs((double)got[i] - (double)want[i]);
    if (a > max_abs) { max_abs = a; max_idx = i; }
    if (got[i] != 0.0f) ++nonzero;
  }
  out[0] = sw > 0.0 ? sqrt(se / sw) : 0.0;
  out[1] = max_abs;
  out[2] = sw > 0.0 ? sqrt(sw / (double)total) : 0.0;
  out[3] = (double)max_idx;
  out[4] = (double)nonzero;
  out[5] = (double)total;
}
