// backend.cpp -- Backend of the device layer over the CUDA kernels, plus a flat
// C cover so non-C++ hosts (and the tests) can drive the same object.
// Mirrors the reference's src/device/backend.cpp: thread-local refusal text
// (:11-17), one concrete backend selected through capability checks (:25-52),
// create() behind the arch guard (:54-62), from_caps() (:64-67),
// would_instantiate() (:69-84).
#include "backend.h"

#include <cstdio>
#include <cstring>

namespace {

thread_local char g_refusal[128] = "";
thread_local int g_launch_status = 0;

class CudaBackend final : public Backend {
 public:
  using Backend::Backend;

  // Tensor-core path = the prefill grouped GEMM. Gate first (the reference's
  // rule: a kernel needing a capability the device lacks is never
  // instantiated), then launch if the plan carries work.
  bool launch_expert_gemm_wmma(const ExpertPlan &plan) override {
    if (!caps_.has_wmma) return false;
    if (!plan.empty()) g_launch_status = knj_moe_ffn_prefill_launch(&plan.args, plan.stream);
    return true;
  }
  // Warp-level path = the decode expert GEMV kernels. Gate = the arch guard.
  bool launch_expert_gemm_simt(const ExpertPlan &plan) override {
    if (!caps_.arch_ok) return false;
    if (!plan.empty()) g_launch_status = knj_moe_ffn_decode_launch(&plan.args, plan.stream);
    return true;
  }
  bool launch_attention(const AttentionPlan &) override { return caps_.arch_ok; }
  void launch_kv_write(const KvWritePlan &) override {}
};

}  // namespace

const char *Backend::knj_last_refusal() { return g_refusal; }
int Backend::knj_last_launch_status() { return g_launch_status; }

std::unique_ptr<Backend> Backend::create() {
  const DeviceCaps caps = knj_probe_host_caps();
  if (!caps.arch_ok) {
    std::snprintf(g_refusal, sizeof g_refusal, "%s", caps.arch_reason ? caps.arch_reason : "arch guard refused");
    return nullptr;
  }
  g_refusal[0] = '\0';
  return std::unique_ptr<Backend>(new CudaBackend(caps));
}

std::unique_ptr<Backend> Backend::from_caps(const DeviceCaps &caps) {
  g_refusal[0] = '\0';
  return std::unique_ptr<Backend>(new CudaBackend(caps));
}

bool Backend::would_instantiate(KnjCap cap) const noexcept {
  if (!knj_cap_available(caps_.gcn_arch, cap)) return false;
  switch (cap) {
    case KnjCap::WmmaF16:
    case KnjCap::TcGen05:
    case KnjCap::Tmem: return caps_.has_wmma;
    case KnjCap::Fp8: return caps_.has_fp8;
    default: return true;
  }
}

// ---- flat C cover -----------------------------------------------------------
extern "C" {

// Returns a Backend* (or null, see knj_backend_last_refusal). Owned by the caller.
void *knj_backend_create(void) { return Backend::create().release(); }
// Fake-device injection: arch string + the three probed flags.
void *knj_backend_from_caps(const char *arch, int has_wmma, int has_fp8, int has_dot_builtin, int arch_ok) {
  DeviceCaps c;
  std::memset(&c, 0, sizeof c);
  if (arch) std::strncpy(c.gcn_arch, arch, sizeof(c.gcn_arch) - 1);
  c.has_wmma = has_wmma != 0;
  c.has_fp8 = has_fp8 != 0;
  c.has_dot_builtin = has_dot_builtin != 0;
  c.wave_size = 32;
  c.arch_ok = arch_ok != 0;
  c.arch_reason = "";
  return Backend::from_caps(c).release();
}
void knj_backend_destroy(void *b) { delete static_cast<Backend *>(b); }
const char *knj_backend_last_refusal(void) { return Backend::knj_last_refusal(); }
int knj_backend_last_launch_status(void) { return Backend::knj_last_launch_status(); }
int knj_backend_would_instantiate(void *b, int cap) {
  return static_cast<Backend *>(b)->would_instantiate(static_cast<KnjCap>(cap)) ? 1 : 0;
}
const char *knj_backend_arch(void *b) { return static_cast<Backend *>(b)->caps().gcn_arch; }
// kind: 0 = tensor-core expert GEMM, 1 = warp-level expert GEMM, 2 = attention gate.
// args may be null (empty plan: gate verdict only, nothing launched).
int knj_backend_launch(void *b, int kind, const knj_moe_ffn_args *args, knj_stream_t stream) {
  ExpertPlan plan;
  if (args) plan.args = *args;
  plan.stream = stream;
  Backend *be = static_cast<Backend *>(b);
  if (kind == 0) return be->launch_expert_gemm_wmma(plan) ? 1 : 0;
  if (kind == 1) return be->launch_expert_gemm_simt(plan) ? 1 : 0;
  return be->launch_attention(AttentionPlan{}) ? 1 : 0;
}
int knj_cap_line(const char *arch, int has_wmma, int has_fp8, int has_dot_builtin, int pk_fma_verified, char *out,
                 size_t cap) {
  DeviceCaps c;
  std::memset(&c, 0, sizeof c);
  if (arch) std::strncpy(c.gcn_arch, arch, sizeof(c.gcn_arch) - 1);
  c.has_wmma = has_wmma != 0;
  c.has_fp8 = has_fp8 != 0;
  c.has_dot_builtin = has_dot_builtin != 0;
  knj_print_cap_line(c, pk_fma_verified != 0, out, cap);
  return 0;
}
int knj_cap_available_c(const char *arch, int cap) { return knj_cap_available(arch, static_cast<KnjCap>(cap)) ? 1 : 0; }
const char *knj_cap_label_c(int cap) { return knj_cap_label(static_cast<KnjCap>(cap)); }
// verdict of the arch guard for explicit strings: 0 ok, 1 refused; *reason set
int knj_check_arch_c(const char *env_arch, const char *built_arch, const char **reason) {
  const KnjArchVerdict v = knj_check_arch(env_arch, built_arch);
  if (reason) *reason = v.reason;
  return v.ok ? 0 : 1;
}

}  // extern "C"
