// device_caps.h -- capability record and arch guard of the device layer, for
// the CUDA (sm_100) build.
//
// Mirrors the reference's src/device/device_caps.h so code written against it
// compiles unchanged: struct DeviceCaps (:57-85, same field names and order),
// enum class KnjCap (:46-53, extended at the END with the CUDA capabilities),
// knj_check_arch (:100-116), knj_build_arch_env (:120-122),
// knj_probe_host_caps (:131-160), knj_cap_available (:168-182), knj_cap_label
// (:186-196), knj_dot_label (:211-215), knj_print_cap_line (:219-231),
// knj_print_doctor_header (:236-252).
//
// Host C++17, no CUDA headers. Runtime facts (memory size, SM count, clock) are
// filled by knj_dev_caps() of the C-ABI (include/knj_device.h).
//
// What changes for CUDA, and only this:
//   * the compiled arch name defaults to "sm_100" (KNJ_ARCH_NAME);
//   * the capability table knows "sm_100": dp4a integer dots, packed half2 fma,
//     the tensor-core path (the field the reference calls has_wmma is true and
//     means "tcgen05 MMA with TMEM accumulators"), fp8; no sdot4 builtin;
//   * the cap line keeps its five fields and their order; the dot field reads
//     "intrinsic(dp4a)" and the last field keeps the reference's key name with
//     the packed-half2-fma verdict as its value.
#ifndef KNJ_DEVICE_CAPS_H
#define KNJ_DEVICE_CAPS_H

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#ifndef KNJ_ARCH_NAME
#define KNJ_ARCH_NAME "sm_100"
#endif
#ifndef KNJ_HAS_WMMA
#define KNJ_HAS_WMMA 1 /* tensor-core path: tcgen05.mma + TMEM */
#endif
#ifndef KNJ_HAS_FP8
#define KNJ_HAS_FP8 1
#endif
#ifndef KNJ_HAS_DOT_ASM
#define KNJ_HAS_DOT_ASM 1 /* dp4a */
#endif

enum class KnjCap {
  Dot4I32I8,     // 4 x s8 dot-accumulate           (dp4a on sm_100)
  Dot8I32I4,     // 8 x s4 dot-accumulate           (exact emulation on sm_100)
  PkFmaF16,      // packed fp16 fused multiply-add  (HFMA2 on sm_100)
  WmmaF16,       // matrix unit with f16/bf16 operands (tcgen05 on sm_100)
  Fp8,           // fp8 matrix operands
  Sdot4Builtin,  // AMD sdot4 builtin: never on CUDA
  // --- CUDA-only capabilities, appended so the reference's values keep their order
  Dp4a,          // the dp4a instruction itself
  TcGen05,       // tcgen05.mma issue
  Tmem,          // tensor memory allocation
  TmaBulk,       // cp.async.bulk + mbarrier transaction counts
};

struct DeviceCaps {
  char gcn_arch[16];  // arch string: "sm_100" here ("gfx1201" / "gfx1031" in the reference)
  bool has_wmma;      // matrix unit present and usable
  bool has_fp8;
  bool has_dot_builtin;  // AMD sdot4 builtin; always false on CUDA
  int wave_size;         // 32
  uint64_t vram_total, vram_usable;
  bool rebar_full_aperture;
  uint32_t sms, clock_khz;
  uint32_t max_streams, num_queue_groups;
  bool arch_ok;             // arch guard verdict
  const char *arch_reason;  // stable text naming the rule that refused; "" when ok
};

struct KnjArchVerdict {
  bool ok;
  const char *reason;
};

// The guard: the environment must NAME the arch the binary was built for.
// Unset is a refusal of its own (exit-code 7 class), a different name is a
// mismatch (exit-code 6 class).
inline KnjArchVerdict knj_check_arch(const char *env_arch, const char *built_arch) {
  if (!env_arch || !*env_arch)
    return {false,
            "KNJ_BUILD_ARCH is not set: a backend that cannot prove which arch "
            "it was built for must not touch the device"};
  if (!built_arch || !*built_arch || std::strcmp(env_arch, built_arch) != 0)
    return {false,
            "arch mismatch: KNJ_BUILD_ARCH disagrees with the compiled backend "
            "arch (built for a different target than the device it is running on)"};
  return {true, ""};
}

inline const char *knj_build_arch_env() { return std::getenv("KNJ_BUILD_ARCH"); }

// Compile-time facts + the environment guard. Device-only fields stay zero.
inline DeviceCaps knj_probe_host_caps() {
  DeviceCaps c;
  std::memset(&c, 0, sizeof c);
  c.has_wmma = KNJ_HAS_WMMA != 0;
  c.has_fp8 = KNJ_HAS_FP8 != 0;
  c.has_dot_builtin = false;
  c.wave_size = 32;
  const KnjArchVerdict v = knj_check_arch(knj_build_arch_env(), KNJ_ARCH_NAME);
  c.arch_ok = v.ok;
  c.arch_reason = v.reason;
  if (v.ok) std::strncpy(c.gcn_arch, KNJ_ARCH_NAME, sizeof(c.gcn_arch) - 1);
  return c;
}

// Is instruction capability `cap` real on arch string `arch`? The two AMD rows
// are kept so a caps record carrying a reference arch string answers as the
// reference does.
inline bool knj_cap_available(const char *arch, KnjCap cap) {
  if (!arch || !*arch) return false;
  const bool sm100 = std::strcmp(arch, "sm_100") == 0;
  const bool g1201 = std::strcmp(arch, "gfx1201") == 0;
  const bool g1031 = std::strcmp(arch, "gfx1031") == 0;
  switch (cap) {
    case KnjCap::Dot4I32I8:
    case KnjCap::Dot8I32I4:
    case KnjCap::PkFmaF16: return sm100 || g1201 || g1031;
    case KnjCap::WmmaF16:
    case KnjCap::Fp8: return sm100 || g1201;
    case KnjCap::Sdot4Builtin: return g1031;
    case KnjCap::Dp4a:
    case KnjCap::TcGen05:
    case KnjCap::Tmem:
    case KnjCap::TmaBulk: return sm100;
  }
  return false;
}

inline const char *knj_cap_label(KnjCap cap) {
  switch (cap) {
    case KnjCap::Dot4I32I8: return "dot4_i32_i8";
    case KnjCap::Dot8I32I4: return "dot8_i32_i4";
    case KnjCap::PkFmaF16: return "pk_fma_f16";
    case KnjCap::WmmaF16: return "wmma_f16";
    case KnjCap::Fp8: return "fp8";
    case KnjCap::Sdot4Builtin: return "sdot4";
    case KnjCap::Dp4a: return "dp4a";
    case KnjCap::TcGen05: return "tcgen05";
    case KnjCap::Tmem: return "tmem";
    case KnjCap::TmaBulk: return "tma_bulk";
  }
  return "unknown";
}

inline const char *knj_dot_label(const DeviceCaps &c) {
  if (c.has_dot_builtin) return "builtin(sdot4)";
  if (std::strncmp(c.gcn_arch, "gfx", 3) == 0) return "asm(v_dot4_i32_i8)";
  if (KNJ_HAS_DOT_ASM) return "intrinsic(dp4a)";
  return "none";
}

// `capabilities  wmma=..  fp8=..  dot=..  smi=lane-split  v_pk_fma_f16=..` --
// five fields, this order, as the reference's doctor output pins them.
inline void knj_print_cap_line(const DeviceCaps &c, bool pk_fma16_verified, char *out, std::size_t cap) {
  std::snprintf(out, cap, "capabilities  wmma=%s  fp8=%s  dot=%s  smi=lane-split  v_pk_fma_f16=%s",
                c.has_wmma ? "on" : "off", c.has_fp8 ? "on" : "off", knj_dot_label(c),
                pk_fma16_verified ? "yes" : "no");
}

inline void knj_print_doctor_header(const DeviceCaps &c, const char *device_name, bool pk_fma16_verified,
                                    char *out, std::size_t cap) {
  char line[160];
  knj_print_cap_line(c, pk_fma16_verified, line, sizeof line);
  std::snprintf(out, cap, "device        %s  %s  %u CU  wave%d\n%s\nrebar         %s\n",
                device_name ? device_name : "(no device)",
                c.gcn_arch[0] ? c.gcn_arch : "(arch guard refused)", c.sms, c.wave_size, line,
                c.rebar_full_aperture ? "full aperture" : "no full aperture");
}

#endif  // KNJ_DEVICE_CAPS_H
