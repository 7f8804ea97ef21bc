// backend.h -- the gated device handle of the device layer (CUDA build).
//
// Mirrors the reference's src/device/backend.h:37-76: Backend::create() (arch
// guarded, nullptr + knj_last_refusal() on refusal), Backend::from_caps()
// (inject a fake device), caps(), would_instantiate(KnjCap), the four launch
// methods, knj_last_refusal().
//
// In the reference ExpertPlan is an empty placeholder and the launch methods
// only answer "would this be permitted". Here ExpertPlan carries the routed
// expert work the Q4_K kernels consume, and the two expert-GEMM launches run
// real kernels when the plan is populated; an EMPTY plan keeps the reference
// behaviour (returns the gate verdict and launches nothing).
#ifndef KNJ_BACKEND_H
#define KNJ_BACKEND_H

#include <cstddef>
#include <cstdint>
#include <memory>

#include "device_caps.h"
#include "knj_device.h"

struct AttentionPlan {};
struct KvWritePlan {};

// One routed MoE-FFN problem. All pointers are DEVICE pointers owned by the
// caller. Layouts as in include/knj_device.h (knj_moe_ffn_args).
struct ExpertPlan {
  knj_moe_ffn_args args{};      // zero-initialised == empty plan
  knj_stream_t stream = nullptr;
  bool empty() const { return args.n_tokens == 0 || args.w_gate == nullptr; }
};

class Backend {
 public:
  static std::unique_ptr<Backend> create();
  static std::unique_ptr<Backend> from_caps(const DeviceCaps &caps);

  const DeviceCaps &caps() const noexcept { return caps_; }
  bool would_instantiate(KnjCap cap) const noexcept;

  // Tensor-core path: prefill grouped GEMM (tcgen05). Refused (false, nothing
  // launched) when the device has no matrix unit.
  virtual bool launch_expert_gemm_wmma(const ExpertPlan &) = 0;
  // SIMT/warp-MMA path: the decode expert GEMV kernels. Gate = the arch guard.
  virtual bool launch_expert_gemm_simt(const ExpertPlan &) = 0;
  virtual bool launch_attention(const AttentionPlan &) = 0;  // gate only: attention is not on this path
  virtual void launch_kv_write(const KvWritePlan &) = 0;     // gate only

  // Status of the last populated-plan launch on this thread (0 = ok).
  static int knj_last_launch_status();
  static const char *knj_last_refusal();

  virtual ~Backend() = default;

 protected:
  explicit Backend(const DeviceCaps &caps) : caps_(caps) {}
  DeviceCaps caps_;
};

#endif  // KNJ_BACKEND_H
