// knj_moe.cu -- the whole MoE-FFN layer as one C-ABI call: the stage sequence
// of the reference's CPU branch (src/model/model.cpp:399-510 Model::moe,
// preceded by the ffn RMSNorm of :631 and followed by the residual add of
// :652), issued as device kernels on one stream with every intermediate in a
// caller-provided workspace.
#include "knj_common.cuh"
#include "knj_q4k.h"

using namespace knj;

namespace {

inline size_t up256(size_t n) { return (n + 255) & ~(size_t)255; }

struct Carve {
  uint8_t *p;
  size_t used = 0;
  explicit Carve(void *base) : p(static_cast<uint8_t *>(base)) {}
  template <typename T>
  T *take(size_t bytes) {
    T *r = p ? reinterpret_cast<T *>(p + used) : nullptr;
    used += up256(bytes);
    return r;
  }
};

struct DecodeWs {
  float *xn, *logits, *pair_w, *A, *Y;
  int32_t *pair_exp, *pair_idx, *pair_cnt, *exp_list, *n_active;
  uint32_t *counter;
  int32_t *status;
  size_t bytes;
};

DecodeWs carve_decode(void *base, int T, int H, int F, int E, int k) {
  Carve c(base);
  DecodeWs w;
  const size_t P = (size_t)T * k;
  w.xn = c.take<float>((size_t)T * H * 4);
  w.logits = c.take<float>((size_t)T * E * 4);
  w.pair_exp = c.take<int32_t>(P * 4);
  w.pair_w = c.take<float>(P * 4);
  w.pair_idx = c.take<int32_t>((size_t)E * T * 4);
  w.pair_cnt = c.take<int32_t>((size_t)E * 4);
  w.exp_list = c.take<int32_t>((size_t)E * 4);
  w.n_active = c.take<int32_t>(16);
  w.counter = c.take<uint32_t>(64 * 4);  // front kernel's completion counters
  w.status = c.take<int32_t>(16);        // [0] gate+up, [1] down: set when a bounded wait gave up
  w.A = c.take<float>(P * F * 4);
  w.Y = c.take<float>(P * H * 4);
  w.bytes = c.used;
  return w;
}

struct PrefillWs {
  float *xn, *logits, *pair_w, *Y;
  int32_t *pair_exp, *pair_idx, *pair_cnt, *exp_list, *n_active, *status;
  void *xh, *ah;
  size_t bytes;
};

PrefillWs carve_prefill(void *base, int T, int H, int F, int E, int k) {
  Carve c(base);
  PrefillWs w;
  const size_t P = (size_t)T * k;
  w.xn = c.take<float>((size_t)T * H * 4);
  w.logits = c.take<float>((size_t)T * E * 4);
  w.pair_exp = c.take<int32_t>(P * 4);
  w.pair_w = c.take<float>(P * 4);
  w.pair_idx = c.take<int32_t>((size_t)E * T * 4);
  w.pair_cnt = c.take<int32_t>((size_t)E * 4);
  w.exp_list = c.take<int32_t>((size_t)E * 4);
  w.n_active = c.take<int32_t>(16);
  w.status = c.take<int32_t>(16);
  w.xh = c.take<void>((size_t)T * H * 2);
  w.ah = c.take<void>(P * F * 2);
  w.Y = c.take<float>(P * H * 4);
  w.bytes = c.used;
  return w;
}

// Device-clock span around a stage of a layer launch while a span ring is recording (knj_spans.cu).
struct StageSpan {
  int h;
  knj_stream_t s;
  StageSpan(const char *name, knj_stream_t st) : h(knj_spans_active() ? knj_span_begin(name, st) : -1), s(st) {}
  ~StageSpan() { if (h >= 0) knj_span_end(h, s); }
};

int check_args(const knj_moe_ffn_args *a, const char *who) {
  KNJ_REQUIRE(a, "%s: null argument block", who);
  KNJ_REQUIRE(a->x && a->w_router && a->w_gate && a->w_up && a->w_down && a->out, "%s: null tensor pointer", who);
  KNJ_REQUIRE(a->n_tokens >= 0 && a->hidden > 0 && a->ffn > 0 && a->n_experts > 0, "%s: bad sizes", who);
  KNJ_REQUIRE(a->hidden % 256 == 0 && a->ffn % 256 == 0, "%s: hidden=%d and ffn=%d must be multiples of 256", who,
              a->hidden, a->ffn);
  KNJ_REQUIRE(a->top_k >= 1 && a->top_k <= 8 && a->top_k <= a->n_experts, "%s: top_k=%d out of range", who, a->top_k);
  KNJ_REQUIRE(a->n_experts <= 256, "%s: at most 256 experts", who);
  KNJ_REQUIRE(a->x_dtype == KNJ_DT_F32 || a->x_dtype == KNJ_DT_BF16, "%s: x must be f32 or bf16", who);
  KNJ_REQUIRE(a->out_dtype == KNJ_DT_F32 || a->out_dtype == KNJ_DT_BF16, "%s: out must be f32 or bf16", who);
  KNJ_REQUIRE(aligned16(a->w_gate) && aligned16(a->w_up) && aligned16(a->w_down) && aligned16(a->w_router),
              "%s: weight bases must be 16-byte aligned", who);
  KNJ_REQUIRE(a->ldx >= a->hidden && a->ldo >= a->hidden, "%s: row strides shorter than hidden", who);
  KNJ_REQUIRE(a->down_format == 0 || a->down_format == 1, "%s: down_format must be 0 (Q4_K) or 1 (Q6_K)", who);
  return KNJ_OK;
}

}  // namespace

extern "C" {

size_t knj_moe_ffn_workspace_bytes(int n_tokens, int hidden, int ffn, int n_experts, int top_k, int mode) {
  if (n_tokens <= 0) return 256;
  if (mode == 1) return carve_prefill(nullptr, n_tokens, hidden, ffn, n_experts, top_k).bytes;
  return carve_decode(nullptr, n_tokens, hidden, ffn, n_experts, top_k).bytes;
}

int knj_moe_ffn_decode_launch(const knj_moe_ffn_args *a, knj_stream_t s) {
  if (a && a->n_tokens == 0) return KNJ_OK;  // an empty batch has no rows to point at
  int rc = check_args(a, "knj_moe_ffn_decode");
  if (rc) return rc;
  const int T = a->n_tokens, H = a->hidden, F = a->ffn, E = a->n_experts, k = a->top_k;
  if (T == 0) return KNJ_OK;
  const size_t need = knj_moe_ffn_workspace_bytes(T, H, F, E, k, 0);
  if (!a->workspace || a->workspace_bytes < need) {
    set_error("knj_moe_ffn_decode: workspace of %zu bytes needed, %zu given", need, a->workspace_bytes);
    return KNJ_E_WORKSPACE;
  }
  KNJ_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255u) == 0, "knj_moe_ffn_decode: workspace must be 256-byte aligned");
  const DecodeWs w = carve_decode(a->workspace, T, H, F, E, k);
  const int P = T * k;

  int32_t *pair_exp = a->tap_pair_exp ? a->tap_pair_exp : w.pair_exp;
  float *pair_w = a->tap_pair_w ? a->tap_pair_w : w.pair_w;
  KNJ_CUDA(cudaMemsetAsync(w.status, 0, 16, as_stream(s)));  // the projections raise it when a bounded wait gives up
  const void *src = w.xn;  // the rows the experts see
  int src_dt = KNJ_DT_F32;
  int64_t src_ld = H;
  if (T <= 64 && H <= 2048 && a->ldx % 8 == 0 && aligned16(a->x)) {
    // decode batch: norm statistics, routing, tables and the normalised rows in one launch
    StageSpan sp("moe-router", s);
    rc = knj_moe_front_launch(a->x, a->x_dtype, a->ldx, a->norm_w, a->rms_eps, a->w_router, a->router_bias, T, H, E, k,
                              w.logits, pair_exp, pair_w, w.pair_idx, T, w.pair_cnt, w.exp_list, w.n_active, w.xn,
                              w.counter, s);
    if (rc) return rc;
  } else {
    // 1. ffn RMSNorm (optional) -> the rows the router and the experts see
    if (a->norm_w) {
      rc = knj_rmsnorm_launch(a->x, a->x_dtype, a->ldx, a->norm_w, a->rms_eps, T, H, w.xn, s);
      if (rc) return rc;
    } else {
      src = a->x;
      src_dt = a->x_dtype;
      src_ld = a->ldx;
      const int64_t esz = src_dt == KNJ_DT_F32 ? 4 : 2;
      KNJ_REQUIRE(aligned16(src) && (src_ld * esz) % 16 == 0, "knj_moe_ffn_decode: rows of x must be 16-byte aligned");
    }
    // 2. route
    rc = knj_router_topk_launch(src, src_dt, src_ld, a->w_router, a->router_bias, T, H, E, k, w.logits, pair_exp, pair_w, s);
    if (rc) return rc;
    // 3. permutation tables
    rc = knj_moe_permute_launch(pair_exp, P, E, T, w.pair_idx, w.pair_cnt, w.exp_list, w.n_active, s);
    if (rc) return rc;
  }
  // gate, up, silu(g)*u
  {
    StageSpan sp("moe-gate", s);  // gate + up + activation fused
    rc = knj_q4k_gateup_launch(src, src_dt, src_ld, a->w_gate, a->w_up, w.pair_idx, w.pair_cnt, nullptr, w.exp_list,
                               w.n_active, nullptr, nullptr, w.A, F, H, H / 256 * KNJ_Q4K_BYTES, T, E, k, w.status, s);
    if (rc) return rc;
  }
  StageSpan sp_down("moe-down", s);  // down projection and the weighted combine (to the end of the launch)
  if (a->down_format == 1) {
    // mixed-format layer: Q6_K down matrices (210-byte superblocks) through their own decode-class projection
    rc = knj_q6k_proj_launch(w.A, a->w_down, w.pair_idx, w.pair_cnt, w.exp_list, w.n_active, w.Y, H, F, T, E, w.status + 1, s);
    if (rc) return rc;
  } else {
    rc = knj_q4k_proj_launch(w.A, KNJ_DT_F32, F, a->w_down, w.pair_idx, w.pair_cnt, nullptr, w.exp_list, w.n_active, w.Y, H,
                             F, F / 256 * KNJ_Q4K_BYTES, T, E, w.status + 1, s);
    if (rc) return rc;
  }
  // weighted combine (+ residual)
  return knj_moe_combine_launch(w.Y, nullptr, pair_exp, pair_w, a->residual ? a->x : nullptr, a->x_dtype, a->ldx,
                                a->out, a->out_dtype, a->ldo, T, H, k, s);
}

int knj_moe_ffn_prefill_launch(const knj_moe_ffn_args *a, knj_stream_t s) {
  if (a && a->n_tokens == 0) return KNJ_OK;
  int rc = check_args(a, "knj_moe_ffn_prefill");
  if (rc) return rc;
  const int T = a->n_tokens, H = a->hidden, F = a->ffn, E = a->n_experts, k = a->top_k;
  KNJ_REQUIRE(H % 128 == 0 && F % 128 == 0, "knj_moe_ffn_prefill: hidden and ffn must be multiples of 128");
  KNJ_REQUIRE(a->down_format == 0 || (a->ffn <= 1024 && !a->fused_combine),
              "knj_moe_ffn_prefill: Q6_K down matrices need ffn <= 1024 and the ordered combine");
  const size_t need = knj_moe_ffn_workspace_bytes(T, H, F, E, k, 1);
  if (!a->workspace || a->workspace_bytes < need) {
    set_error("knj_moe_ffn_prefill: workspace of %zu bytes needed, %zu given", need, a->workspace_bytes);
    return KNJ_E_WORKSPACE;
  }
  KNJ_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255u) == 0, "knj_moe_ffn_prefill: workspace must be 256-byte aligned");
  const PrefillWs w = carve_prefill(a->workspace, T, H, F, E, k);
  const int P = T * k;

  const void *src = a->x;
  int src_dt = a->x_dtype;
  int64_t src_ld = a->ldx;
  if (a->norm_w) {
    rc = knj_rmsnorm_launch(a->x, a->x_dtype, a->ldx, a->norm_w, a->rms_eps, T, H, w.xn, s);
    if (rc) return rc;
    src = w.xn;
    src_dt = KNJ_DT_F32;
    src_ld = H;
  }
  int32_t *pair_exp = a->tap_pair_exp ? a->tap_pair_exp : w.pair_exp;
  float *pair_w = a->tap_pair_w ? a->tap_pair_w : w.pair_w;
  KNJ_CUDA(cudaMemsetAsync(w.status, 0, 16, as_stream(s)));  // the GEMMs raise it when a bounded wait gives up
  {
    StageSpan sp("moe-router", s);
    rc = knj_router_topk_launch(src, src_dt, src_ld, a->w_router, a->router_bias, T, H, E, k, w.logits, pair_exp, pair_w, s);
    if (rc) return rc;
  }
  {
    StageSpan sp("moe-gather", s);  // permutation tables and fp16 rows (rows are gathered inside the GEMM)
    // long pair lists take the counting-sort form; its scratch is the activation buffer, which is written later
    rc = knj_moe_permute_ws_launch(pair_exp, P, E, T, w.pair_idx, w.pair_cnt, w.exp_list, w.n_active, w.ah,
                                   (size_t)P * F * 2, s);
    if (rc) return rc;
    rc = knj_to_f16_launch(src, src_dt, src_ld, T, H, w.xh, s);
    if (rc) return rc;
  }
  {
    StageSpan sp("moe-gate", s);  // gate + up + activation fused
    rc = knj_q4k_gateup_tc_launch(w.xh, a->w_gate, a->w_up, w.pair_idx, w.pair_cnt, nullptr, w.ah, F, H,
                                  H / 256 * KNJ_Q4K_BYTES, T, E, k, P, w.status, s);
    if (rc) return rc;
  }
  if (a->fused_combine) {
    // down GEMM with the weighted combine in its epilogue: the token's sum starts from the residual (or zero) in
    // f32 and receives its k rows as vector reductions; no per-pair rows exist. The f32 sums sit where the
    // per-pair rows would (or directly in a dense f32 output).
    const bool direct = a->out_dtype == KNJ_DT_F32 && a->ldo == H;
    float *acc = direct ? static_cast<float *>(a->out) : w.Y;
    {
      StageSpan sp("moe-down", s);
      rc = knj_moe_acc_init_launch(a->x, a->x_dtype, a->ldx, a->residual, T, H, acc, s);
      if (rc) return rc;
      rc = knj_q4k_down_combine_tc_launch(w.ah, a->w_down, w.pair_idx, w.pair_cnt, nullptr, pair_w, k, acc, H, F,
                                          F / 256 * KNJ_Q4K_BYTES, T, E, P, w.status, s);
      if (rc) return rc;
    }
    if (direct) return KNJ_OK;
    StageSpan sp("moe-scatter", s);
    return knj_moe_acc_finish_launch(acc, a->out, a->out_dtype, a->ldo, T, H, s);
  }
  {
    StageSpan sp("moe-down", s);
    rc = a->down_format == 1
             ? knj_q6k_down_tc_launch(w.ah, a->w_down, w.pair_idx, w.pair_cnt, nullptr, w.Y, H, F, T, E, P, w.status, s)
             : knj_q4k_down_tc_launch(w.ah, a->w_down, w.pair_idx, w.pair_cnt, nullptr, w.Y, H, F, F / 256 * KNJ_Q4K_BYTES, T, E,
                                      P, w.status, s);
    if (rc) return rc;
  }
  StageSpan sp("moe-scatter", s);
  return knj_moe_combine_launch(w.Y, nullptr, pair_exp, pair_w, a->residual ? a->x : nullptr, a->x_dtype, a->ldx,
                                a->out, a->out_dtype, a->ldo, T, H, k, s);
}

int knj_moe_ffn_status(const knj_moe_ffn_args *a, int mode, knj_stream_t s) {
  int rc = check_args(a, "knj_moe_ffn_status");
  if (rc) return rc;
  if (a->n_tokens == 0) return KNJ_OK;
  KNJ_REQUIRE(a->workspace && (mode == 0 || mode == 1), "knj_moe_ffn_status: no workspace or unknown mode %d", mode);
  const int T = a->n_tokens, H = a->hidden, F = a->ffn, E = a->n_experts, k = a->top_k;
  const int32_t *dev_words = mode == 1 ? carve_prefill(a->workspace, T, H, F, E, k).status : carve_decode(a->workspace, T, H, F, E, k).status;
  int32_t words[4] = {0, 0, 0, 0};
  KNJ_CUDA(cudaMemcpyAsync(words, dev_words, sizeof(words), cudaMemcpyDeviceToHost, as_stream(s)));
  KNJ_CUDA(cudaStreamSynchronize(as_stream(s)));
  if (words[0] != 0 || words[1] != 0) {
    set_error("knj_moe_ffn: a bounded device wait gave up in the %s launch (gate+up %d, down %d)", mode == 1 ? "prefill" : "decode",
              words[0], words[1]);
    return KNJ_E_TIMEOUT;
  }
  return KNJ_OK;
}

}  // extern "C"
