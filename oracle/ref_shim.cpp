// ref_shim.cpp -- C entry points around the REFERENCE's own CPU sources.
//
// TEST INFRASTRUCTURE ONLY. This file is compiled together with the reference
// sources where they lie in the mounted reference tree (see oracle/Makefile,
// target `ref`); none of those sources is copied into this repository. The
// result, oracle/_ref/libknj_ref.so, is used to
//   * validate oracle/knj_oracle.c (the restatement) bit for bit,
//   * generate the golden vectors under tests/golden/,
//   * serve as the timed CPU baseline (kind "reference") in bench.py.
//
// Reference translation units linked in, unmodified:
//   src/loader/dequant.cpp   dequant_row_f32 / dequant_dot_f32 / fp16_to_fp32
//   src/loader/gguf.cpp      ggml_type_block_weights / _bytes / _name
//   src/util/parallel.cpp    knj::ThreadPool
// Reference headers used inline: kernels/knj_q4k.h, tests/host_oracle.h.
//
// knj::Model::moe itself is a private method of a class that can only be
// constructed from a complete GGUF model file, and no model file exists here.
// ref_moe() below therefore walks the same stages as
// src/model/model.cpp:399-510 but performs every weight access through the
// reference's PUBLIC functions (dequant_dot_f32 for one row, dequant_row_f32
// per 256-block for several rows, as src/model/model.cpp:349-364 does) and
// splits output columns over the reference ThreadPool with the reference's
// chunk rule min(n_out, total*4) (src/model/model.cpp:372-379).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <vector>

#include "kernels/knj_q4k.h"
#include "src/loader/dequant.h"
#include "src/util/parallel.h"
#include "tests/host_oracle.h"

namespace {

std::unique_ptr<knj::ThreadPool> g_pool;
int g_pool_threads = -1;

knj::ThreadPool& pool(int threads) {
  if (!g_pool || g_pool_threads != threads) {
    g_pool.reset(new knj::ThreadPool(threads));
    g_pool_threads = threads;
  }
  return *g_pool;
}

// One weight matrix times m activation rows, through the reference decoders.
void ref_matmul(knj::ThreadPool& tp, knj::GgmlType type, const uint8_t* base, int n_in, int n_out,
                const float* x, int m, int ldx, float* y, int ldy) {
  const uint64_t bw = knj::ggml_type_block_weights(type);
  const uint64_t bb = knj::ggml_type_block_bytes(type);
  const uint64_t stride = knj::column_stride_bytes(type, (uint64_t)n_in);
  auto columns = [&](int j0, int j1) {
    std::vector<float> stage(bw == 1 ? (size_t)n_in : 256);
    for (int j = j0; j < j1; ++j) {
      const uint8_t* src = base + (uint64_t)j * stride;
      if (bw == 1) {
        knj::dequant_row_f32(type, src, stage.data(), (uint64_t)n_in);
        for (int r = 0; r < m; ++r) {
          float acc = 0.0f;
          for (int i = 0; i < n_in; ++i) acc += stage[(size_t)i] * x[(size_t)r * ldx + i];
          y[(size_t)r * ldy + j] = acc;
        }
      } else if (m == 1) {
        y[j] = knj::dequant_dot_f32(type, src, x, (uint64_t)n_in);
      } else {
        for (int r = 0; r < m; ++r) y[(size_t)r * ldy + j] = 0.0f;
        for (uint64_t b = 0; b < (uint64_t)n_in / bw; ++b) {
          knj::dequant_row_f32(type, src + b * bb, stage.data(), bw);
          for (int r = 0; r < m; ++r) {
            const float* xr = x + (size_t)r * ldx + b * bw;
            float acc = 0.0f;
            for (uint64_t l = 0; l < bw; ++l) acc += stage[l] * xr[l];
            y[(size_t)r * ldy + j] += acc;
          }
        }
      }
    }
  };
  const uint64_t work = (uint64_t)n_in * (uint64_t)n_out * (uint64_t)m;
  if (work < (1ull << 16) || tp.total() <= 1) {
    columns(0, n_out);
    return;
  }
  const int nt = std::min<int>(n_out, tp.total() * 4);
  const int per = (n_out + nt - 1) / nt;
  tp.for_each(nt, [&](int t) { columns(t * per, std::min(n_out, (t + 1) * per)); });
}

inline float ref_silu(float v) { return v / (1.0f + std::exp(-v)); }

}  // namespace

extern "C" {

float ref_fp16_to_fp32(uint16_t h) { return knj::fp16_to_fp32(h); }
float ref_half_bits_to_float(uint16_t h) { return knj_half_bits_to_float(h); }
float ref_host_oracle_h2f(uint16_t h) { return knj_ref::h2f(h); }

void ref_dequant_row_q4k(const uint8_t* src, float* dst, uint64_t n) {
  knj::dequant_row_f32(knj::GgmlType::Q4_K, src, dst, n);
}
void ref_dequant_row_q6k(const uint8_t* src, float* dst, uint64_t n) {
  knj::dequant_row_f32(knj::GgmlType::Q6_K, src, dst, n);
}
float ref_dequant_dot_q4k(const uint8_t* src, const float* x, uint64_t n) {
  return knj::dequant_dot_f32(knj::GgmlType::Q4_K, src, x, n);
}
float ref_q4k_weight(const uint8_t* blk, int r) { return knj_q4k_weight(blk, r); }
float ref_q6k_weight(const uint8_t* blk, int r) { return knj_q6k_weight(blk, r); }
void ref_q4k_span16(const uint8_t* blk, int r0, float* out) { knj_q4k_span16(blk, r0, out); }
void ref_q4k_scale_min(const uint8_t* sc, int j, uint8_t* d, uint8_t* m) {
  knj_q4k_scale_min(sc, j, d, m);
}

void ref_gemm_w4_reference(const uint8_t* Bq, const int8_t* Act, float* C, int M, int N, int K) {
  knj_ref::gemm_w4_reference(Bq, Act, C, M, N, K);
}
void ref_deinterleave_activations(const int8_t* Act, uint32_t* Out, int M, int K) {
  knj_ref::deinterleave_activations(Act, Out, M, K);
}
void ref_compare(const float* got, const float* want, int M, int N, double* out) {
  const knj_ref::ErrorStats s = knj_ref::compare(got, want, M, N);
  out[0] = s.rel_rmse; out[1] = s.max_abs; out[2] = s.out_rms;
  out[3] = (double)s.max_idx; out[4] = (double)s.nonzero; out[5] = (double)s.total;
}

// Q4_K matrix [n_out rows of n_in] times m rows, on `threads` host threads.
void ref_matmul_q4k(const uint8_t* W, int n_in, int n_out, const float* x, int m, int ldx, float* y,
                    int ldy, int threads) {
  ref_matmul(pool(threads), knj::GgmlType::Q4_K, W, n_in, n_out, x, m, ldx, y, ldy);
}

// The MoE branch (stages of src/model/model.cpp:399-510) over reference
// decoders. Wr is bf16 [E][H]; Wg/Wu Q4_K [E][F][H/256][144]; Wd Q4_K
// [E][H][F/256][144]. chosen/weight taps [m][K] may be null.
void ref_moe(const uint16_t* Wr_bf16, const uint8_t* Wg, const uint8_t* Wu, const uint8_t* Wd,
             const float* hx, int m, int H, int E, int K, int F, float* out, int32_t* chosen_tap,
             float* weight_tap, int threads) {
  knj::ThreadPool& tp = pool(threads);
  std::vector<float> rlog((size_t)m * E), probs((size_t)E);
  ref_matmul(tp, knj::GgmlType::BF16, reinterpret_cast<const uint8_t*>(Wr_bf16), H, E, hx, m, H,
             rlog.data(), E);
  std::vector<std::vector<int32_t>> ex_tok((size_t)E);
  std::vector<std::vector<float>> ex_w((size_t)E);
  std::vector<int> pick((size_t)K);
  for (int t = 0; t < m; ++t) {
    const float* lg = rlog.data() + (size_t)t * E;
    float mx = lg[0];
    for (int e = 1; e < E; ++e) mx = std::max(mx, lg[e]);
    float sum = 0.0f;
    for (int e = 0; e < E; ++e) { probs[e] = std::exp(lg[e] - mx); sum += probs[e]; }
    for (int e = 0; e < E; ++e) probs[e] /= sum;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      for (int e = 0; e < E; ++e) {
        bool used = false;
        for (int q = 0; q < k; ++q) used = used || pick[q] == e;
        if (used) continue;
        if (best < 0 || probs[e] > probs[best]) best = e;
      }
      pick[k] = best;
    }
    float keep = 0.0f;
    for (int k = 0; k < K; ++k) keep += probs[pick[k]];
    const float inv = keep > 0.0f ? 1.0f / keep : 0.0f;
    for (int k = 0; k < K; ++k) {
      ex_tok[pick[k]].push_back(t);
      ex_w[pick[k]].push_back(probs[pick[k]] * inv);
      if (chosen_tap) chosen_tap[(size_t)t * K + k] = pick[k];
      if (weight_tap) weight_tap[(size_t)t * K + k] = probs[pick[k]] * inv;
    }
  }
  std::fill(out, out + (size_t)m * H, 0.0f);
  std::vector<float> gat((size_t)m * H), yg((size_t)m * F), yu((size_t)m * F), yd((size_t)m * H);
  const uint64_t gu_slab = knj::tensor_bytes(knj::GgmlType::Q4_K, (uint64_t)H, (uint64_t)F);
  const uint64_t dn_slab = knj::tensor_bytes(knj::GgmlType::Q4_K, (uint64_t)F, (uint64_t)H);
  for (int e = 0; e < E; ++e) {
    const int cnt = (int)ex_tok[e].size();
    if (cnt == 0) continue;
    for (int r = 0; r < cnt; ++r)
      std::memcpy(gat.data() + (size_t)r * H, hx + (size_t)ex_tok[e][r] * H, sizeof(float) * H);
    ref_matmul(tp, knj::GgmlType::Q4_K, Wg + e * gu_slab, H, F, gat.data(), cnt, H, yg.data(), F);
    ref_matmul(tp, knj::GgmlType::Q4_K, Wu + e * gu_slab, H, F, gat.data(), cnt, H, yu.data(), F);
    for (size_t i = 0, n = (size_t)cnt * F; i < n; ++i) yg[i] = ref_silu(yg[i]) * yu[i];
    ref_matmul(tp, knj::GgmlType::Q4_K, Wd + e * dn_slab, F, H, yg.data(), cnt, F, yd.data(), H);
    for (int r = 0; r < cnt; ++r) {
      const float wt = ex_w[e][r];
      float* dst = out + (size_t)ex_tok[e][r] * H;
      const float* src = yd.data() + (size_t)r * H;
      for (int i = 0; i < H; ++i) dst[i] += wt * src[i];
    }
  }
}

int ref_hardware_threads() { return (int)std::max(1u, std::thread::hardware_concurrency()); }

}  // extern "C"
