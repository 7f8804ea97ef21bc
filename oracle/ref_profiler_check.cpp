// ref_profiler_check.cpp -- test infrastructure, not part of the shipped library.
//
// Feeds the device spans this library records around the stages of a layer launch (knj_spans_*, the CUDA event
// ring behind the reference's "dev" column) into the REFERENCE's Profiler (src/profiler/profiler.h:98-137,
// device_span at :125), compiled from src/profiler/profiler.cpp and src/platform/memprobe.cpp where they lie, and
// checks what its reports then say: the domain is Device, every flushed span was counted, the rows carry the CPU
// path's stage names (src/model/model.cpp:408-500) with non-zero device time, nothing was dropped.
//
// Built by `make -C oracle ref` into oracle/_ref/knj_ref_profiler_check (needs the reference tree at build time
// only); run on a machine with a GPU by tests/test_gpu_spans.py. Exit code = number of failed checks.
#include "src/profiler/profiler.h"

#include "knj_device.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {

int g_checks = 0, g_failed = 0;
void check(bool ok, const char *what) {
  ++g_checks;
  if (!ok) {
    ++g_failed;
    std::printf("  FAIL  %s\n", what);
  }
}
#define CHECK(x) check((x), #x)
#define OK(call) check((call) == KNJ_OK, #call)

uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

// pseudo-random Q4_K matrices with sane super-block factors (fp16 d = 2^-6, dmin = 2^-8)
std::vector<uint8_t> q4k_bytes(size_t n_blocks, uint32_t seed) {
  std::vector<uint8_t> w(n_blocks * 144);
  uint32_t s = seed;
  for (auto &b : w) {
    s = s * 1664525u + 1013904223u;
    b = (uint8_t)(s >> 24);
  }
  for (size_t i = 0; i < n_blocks; ++i) {
    const uint16_t d = 0x2400, dmin = 0x1c00;
    std::memcpy(&w[i * 144], &d, 2);
    std::memcpy(&w[i * 144 + 2], &dmin, 2);
  }
  return w;
}

void *to_device(const void *src, size_t bytes) {
  void *d = nullptr;
  if (knj_malloc(&d, bytes) != KNJ_OK || knj_memcpy_h2d(d, src, bytes) != KNJ_OK) {
    std::printf("device set-up failed: %s\n", knj_last_error_string());
    std::exit(78);
  }
  return d;
}

struct Seen {
  knj::Profiler *p;
  int n = 0;
  std::vector<std::string> names;
};

}  // namespace

int main() {
  int n_dev = 0;
  if (knj_dev_count(&n_dev) != KNJ_OK || n_dev == 0) {
    std::printf("no CUDA device: nothing checked\n");
    return 77;
  }
  OK(knj_dev_open(0));
  const int E = 8, H = 512, F = 256, K = 2, T = 4, steps = 3;
  std::vector<float> x((size_t)T * H);
  for (size_t i = 0; i < x.size(); ++i) x[i] = 0.01f * (float)((int)(i * 37 % 201) - 100);
  std::vector<uint16_t> router((size_t)E * H);
  for (size_t i = 0; i < router.size(); ++i) router[i] = f32_to_bf16(0.02f * (float)((int)(i * 53 % 101) - 50) / 50.0f);
  const auto gate = q4k_bytes((size_t)E * F * (H / 256), 1), up = q4k_bytes((size_t)E * F * (H / 256), 2),
             down = q4k_bytes((size_t)E * H * (F / 256), 3);
  knj_moe_ffn_args a{};
  a.n_tokens = T; a.hidden = H; a.ffn = F; a.n_experts = E; a.top_k = K;
  a.x_dtype = KNJ_DT_F32; a.x = to_device(x.data(), x.size() * 4); a.ldx = H;
  a.w_router = static_cast<const uint16_t *>(to_device(router.data(), router.size() * 2));
  a.w_gate = static_cast<const uint8_t *>(to_device(gate.data(), gate.size()));
  a.w_up = static_cast<const uint8_t *>(to_device(up.data(), up.size()));
  a.w_down = static_cast<const uint8_t *>(to_device(down.data(), down.size()));
  a.rms_eps = 1e-6f;
  void *out = nullptr;
  OK(knj_malloc(&out, (size_t)T * H * 4));
  a.out = out; a.out_dtype = KNJ_DT_F32; a.ldo = H;
  a.workspace_bytes = knj_moe_ffn_workspace_bytes(T, H, F, E, K, 0);
  OK(knj_malloc(&a.workspace, a.workspace_bytes));

  knj_stream_t stream = nullptr;  // the default stream
  OK(knj_spans_enable(4096));
  OK(knj_spans_epoch(stream));
  for (int i = 0; i < steps; ++i) OK(knj_moe_ffn_decode_launch(&a, stream));
  OK(knj_dev_sync());
  OK(knj_moe_ffn_status(&a, 0, stream));

  knj::Profiler &p = knj::Profiler::get();
  knj::ProfileConfig cfg;
  cfg.on = true;
  cfg.format = "table";
  cfg.warmup_steps = 0;
  p.configure(cfg);
  p.enable_device_backend();
  CHECK(p.domain() == knj::ClockDomain::Device);
  Seen seen{&p};
  OK(knj_spans_flush(
      [](const char *name, uint64_t a_ns, uint64_t b_ns, int st, void *user) {
        Seen *s = static_cast<Seen *>(user);
        s->p->device_span(name, a_ns, b_ns, st);
        s->names.emplace_back(name);
        if (b_ns >= a_ns) ++s->n;
      },
      &seen));
  p.set_device_dropped(knj_spans_dropped());
  for (int i = 0; i < steps; ++i) p.step_done();
  CHECK(seen.n == (int)seen.names.size() && seen.n >= 3 * steps);  // router, gate, down at least, per step
  CHECK(p.device_spans() == (uint64_t)seen.n);
  CHECK(p.device_dropped() == 0);

  // what the reference's own report writers make of them
  char path[] = "/tmp/knj_profile_XXXXXX";
  const int fd = mkstemp(path);
  CHECK(fd >= 0);
  std::FILE *f = fdopen(fd, "w+");
  p.report_table(f);
  p.report_json(f);
  std::fflush(f);
  std::rewind(f);
  std::string text;
  char buf[4096];
  size_t got;
  while ((got = std::fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, got);
  std::fclose(f);
  std::remove(path);
  std::printf("%s\n", text.c_str());
  CHECK(text.find("moe-router") != std::string::npos);
  CHECK(text.find("moe-gate") != std::string::npos);
  CHECK(text.find("moe-down") != std::string::npos);
  CHECK(text.find(knj::clock_domain_name(knj::ClockDomain::Device)) != std::string::npos);
  OK(knj_spans_disable());
  std::printf("reference Profiler fed from the device span ring: %d spans, %d checks, %d failed\n", seen.n, g_checks, g_failed);
  return g_failed;
}
