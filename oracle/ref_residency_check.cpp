// ref_residency_check.cpp -- test infrastructure, not part of the shipped library.
//
// Constructs the REFERENCE's residency state machine (ResidencyManager, src/residency/residency.h:254-369,
// compiled from src/residency/residency.cpp where it lies) over this repository's CUDA gates
// (include/knj_residency.h: slot pool, copy engine with a file tier, pinned arena) and drives it the way the
// reference's own unit test drives it over fakes (tests/unit/test_c9_residency.cpp:594-640: one manager, one set
// of gates, tick() as the only place a completion is seen) -- but with real asynchronous copies: a backing file
// on disk, pread into pinned memory, cudaMemcpyAsync into device slots. Checked: a demanded expert walks
// NVME -> RAM -> VRAM and is `ready` only when the slot's copies have finished; the slot then holds the file's
// bytes; with the pool full a further demand stays not-ready and goes to the fallback sink without blocking;
// after an eviction the waiting expert gets the slot; a reload reproduces the same bytes.
//
// Built by `make -C oracle ref` into oracle/_ref/knj_ref_residency_check (needs the reference tree at build
// time only); run on a machine with a GPU by tests/test_gpu_residency.py. Exit code = number of failed checks.
#include "src/residency/residency.h"  // the reference's, first: knj_residency.h then declares only the factories

#include "knj_residency.h"

#include <cuda_runtime.h>
#include <unistd.h>

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

constexpr uint64_t kExpertBytes = 256 * 1024;
constexpr int kExperts = 6, kSlots = 3;

uint8_t pattern(uint64_t file_offset) { return (uint8_t)((file_offset * 131u + 7u + (file_offset >> 18)) & 0xffu); }

struct Fallback final : knj::FallbackSink {
  int experts = 0, kv = 0;
  void expert_unavailable(knj::ExpertId, knj::Residency) override { ++experts; }
  void kv_unavailable(knj::KvPageId, knj::Residency) override { ++kv; }
};
struct Telemetry final : knj::TelemetrySink {
  int transitions = 0, misses = 0;
  void on_transition(const knj::TransitionEvent &) override { ++transitions; }
  void on_deadline_missed(const knj::TransitionEvent &, uint64_t) override { ++misses; }
};

uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

// tick until `done()` or the bound runs out (real copies complete in wall time, not in ticks)
template <class F>
bool tick_until(knj::ResidencyManager &m, F done, int max_ticks = 20000) {
  for (int i = 0; i < max_ticks; ++i) {
    m.begin_layer(0);  // one layer's experts: the layer index never moves backwards
    m.tick();
    if (done()) return true;
    usleep(100);
  }
  return false;
}

// the device slot that holds exactly the bytes of expert e's extent, or -1
int slot_with_expert(knj::SlotAllocator &slots, int e) {
  std::vector<uint8_t> host(kExpertBytes);
  for (int h = 0; h < kSlots; ++h) {
    void *p = slots.vram_ptr(h);
    if (!p || slots.byte_size(h) != kExpertBytes) continue;
    if (cudaMemcpy(host.data(), p, kExpertBytes, cudaMemcpyDeviceToHost) != cudaSuccess) continue;
    bool same = true;
    for (uint64_t i = 0; i < kExpertBytes && same; ++i) same = host[i] == pattern((uint64_t)e * kExpertBytes + i);
    if (same) return h;
  }
  return -1;
}

}  // namespace

int main() {
  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
    std::printf("no CUDA device: nothing checked\n");
    return 77;
  }
  cudaSetDevice(0);
  // backing store
  char path[] = "/tmp/knj_residency_XXXXXX";
  const int fd = mkstemp(path);
  if (fd < 0) return 78;
  {
    std::vector<uint8_t> all(kExpertBytes * kExperts);
    for (uint64_t i = 0; i < all.size(); ++i) all[i] = pattern(i);
    if (write(fd, all.data(), all.size()) != (ssize_t)all.size()) return 78;
    close(fd);
  }
  {
    auto arena = knj::make_cuda_host_arena();
    auto slots = knj::make_cuda_slot_allocator(kSlots, kExpertBytes);
    auto engine = knj::make_cuda_transfer_engine(path, slots.get());
    Fallback fb;
    Telemetry tel;
    knj::ResidencyManager::Config cfg;
    cfg.slots = slots.get();
    cfg.transfer = engine.get();
    cfg.arena = arena.get();
    cfg.fallback = &fb;
    cfg.telemetry = &tel;
    cfg.now_ns = &now_ns;
    cfg.demand_deadline_ticks = 1;
    cfg.prefetch_ttl_ticks = 4;
    knj::ResidencyManager m(cfg);
    auto id = [](int e) { return knj::ExpertId{0u, (uint32_t)e}; };
    for (int e = 0; e < kExperts; ++e) m.register_expert(id(e), knj::BackingExtent{(uint64_t)e * kExpertBytes, kExpertBytes});
    CHECK(m.n_experts() == (size_t)kExperts);
    CHECK(m.locate(id(0)) == knj::Residency::NVME_RESIDENT);
    CHECK(!m.ready(id(0)));

    // one expert through both hops
    m.request(id(0), knj::KVTier::VRAM);
    CHECK(m.locate(id(0)) == knj::Residency::LOADING_NVME);
    CHECK(!m.ready(id(0)));  // issued is not ready
    CHECK(tick_until(m, [&] { return m.ready(id(0)); }));
    CHECK(m.locate(id(0)) == knj::Residency::VRAM_RESIDENT);
    CHECK(slot_with_expert(*slots, 0) >= 0);
    CHECK(m.kernel_view().ready(id(0)));

    // fill the pool
    m.request(id(1), knj::KVTier::VRAM);
    m.request(id(2), knj::KVTier::VRAM);
    CHECK(tick_until(m, [&] { return m.ready(id(1)) && m.ready(id(2)); }));
    CHECK(slot_with_expert(*slots, 1) >= 0 && slot_with_expert(*slots, 2) >= 0);

    // a fourth demand: no room -> stays in RAM, not ready, the contribution goes to the fallback sink; nothing blocks
    const int fb_before = fb.experts;
    CHECK(!m.demand_or_fallback(id(3)));
    CHECK(fb.experts == fb_before + 1);
    CHECK(tick_until(m, [&] { return m.locate(id(3)) == knj::Residency::RAM_RESIDENT; }));
    for (int i = 0; i < 50; ++i) m.tick();
    CHECK(!m.ready(id(3)));
    CHECK(m.locate(id(3)) == knj::Residency::RAM_RESIDENT);
    CHECK(m.ready(id(0)) && m.ready(id(1)) && m.ready(id(2)));  // nothing in use was evicted to make room

    // eviction is the caller's decision; afterwards the waiting expert gets the slot
    m.demote(id(0));
    CHECK(m.locate(id(0)) == knj::Residency::EVICTING_VRAM);
    CHECK(tick_until(m, [&] { return m.locate(id(0)) == knj::Residency::RAM_RESIDENT; }));
    CHECK(!m.ready(id(0)));
    m.request(id(3), knj::KVTier::VRAM);
    CHECK(tick_until(m, [&] { return m.ready(id(3)); }));
    CHECK(slot_with_expert(*slots, 3) >= 0);
    CHECK(slot_with_expert(*slots, 0) < 0);

    // pinning refuses eviction
    m.pin(id(1));
    CHECK(m.locate(id(1)) == knj::Residency::PINNED);
    const uint64_t refused = m.refused_demotions();
    m.demote(id(1));
    CHECK(m.refused_demotions() == refused + 1 && m.ready(id(1)));
    m.unpin(id(1));

    // a reload reproduces the same bytes: all the way down, then up again
    m.demote(id(2));
    CHECK(tick_until(m, [&] { return m.locate(id(2)) == knj::Residency::RAM_RESIDENT; }));
    m.demote(id(2));
    CHECK(tick_until(m, [&] { return m.locate(id(2)) == knj::Residency::NVME_RESIDENT; }));
    m.request(id(2), knj::KVTier::VRAM);
    CHECK(tick_until(m, [&] { return m.ready(id(2)); }));
    CHECK(slot_with_expert(*slots, 2) >= 0);

    // a prefetch lands as PREFETCHED and is consumed by a demand
    m.demote(id(3));
    CHECK(tick_until(m, [&] { return m.locate(id(3)) == knj::Residency::RAM_RESIDENT; }));
    m.prefetch(id(4), knj::KVTier::VRAM, knj::PrefetchPriority::NORMAL);
    CHECK(tick_until(m, [&] { return m.locate(id(4)) == knj::Residency::PREFETCHED; }));
    CHECK(m.demand(id(4), knj::KVTier::VRAM));
    CHECK(slot_with_expert(*slots, 4) >= 0);

    CHECK(tel.transitions > 0 && (uint64_t)tel.transitions == m.transitions());
    CHECK(knj::ResidencyManager::blocking_transfer_calls() == 0);
    m.reset();
    CHECK(m.locate(id(1)) == knj::Residency::NVME_RESIDENT);
  }
  unlink(path);
  std::printf("reference ResidencyManager over the CUDA gates: %d checks, %d failed\n", g_checks, g_failed);
  return g_failed;
}
