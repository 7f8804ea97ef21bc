// knj_spans.cu -- device-clock spans of the layer launches for a host profiler.
//
// The reference's profiler takes device rows through
// Profiler::device_span(name, start_ns, end_ns, stream) (src/profiler/profiler.h:98-125):
// offsets from ONE epoch event on the same stream, handed over at flush time,
// never inside the step loop, with a count of the spans its event ring could not
// hold (set_device_dropped, :133-137). This file is that event ring for CUDA:
// knj_spans_epoch() marks the epoch, the layer launchers bracket their stages
// with knj_span_begin/end while recording is on (names as the CPU path's rows,
// src/model/model.cpp:408-500: moe-router, moe-gather, moe-gate, moe-act,
// moe-down, moe-scatter; fused stages carry the name of their dominant part),
// and knj_spans_flush() synchronises once and calls back with nanosecond offsets.
// Launches made while a stream is being captured into a graph record nothing:
// events inside a capture cannot be timed.
#include <vector>

#include "knj_common.cuh"

using namespace knj;

namespace {

struct SpanRec {
  char name[32];
  cudaEvent_t a = nullptr, b = nullptr;
  bool closed = false;
};

struct SpanRing {
  bool on = false;
  cudaEvent_t epoch = nullptr;
  bool have_epoch = false;
  std::vector<SpanRec> recs;
  size_t used = 0;
  uint64_t dropped = 0;
};

SpanRing g_ring;

bool capturing(cudaStream_t st) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return cs != cudaStreamCaptureStatusNone;
}

}  // namespace

extern "C" {

int g_span_capacity = 0;  // spans beyond it are counted as dropped

int knj_spans_enable(int capacity) {
  KNJ_REQUIRE(capacity >= 1 && capacity <= (1 << 20), "knj_spans_enable: capacity %d out of range", capacity);
  if (!g_ring.epoch) KNJ_CUDA(cudaEventCreate(&g_ring.epoch));
  const size_t old = g_ring.recs.size();
  if ((size_t)capacity > old) {  // a smaller ring keeps the events it has and uses fewer of them
    g_ring.recs.resize(capacity);
    for (size_t i = old; i < g_ring.recs.size(); ++i) {
      KNJ_CUDA(cudaEventCreate(&g_ring.recs[i].a));
      KNJ_CUDA(cudaEventCreate(&g_ring.recs[i].b));
    }
  }
  g_span_capacity = capacity;
  g_ring.used = 0;
  g_ring.dropped = 0;
  g_ring.have_epoch = false;
  g_ring.on = true;
  return KNJ_OK;
}

int knj_spans_disable(void) {
  g_ring.on = false;
  return KNJ_OK;
}

int knj_spans_active(void) { return g_ring.on ? 1 : 0; }

int knj_spans_epoch(knj_stream_t s) {
  KNJ_REQUIRE(g_ring.on, "knj_spans_epoch: recording is off");
  cudaStream_t st = as_stream(s);
  KNJ_REQUIRE(!capturing(st), "knj_spans_epoch: the stream is being captured");
  KNJ_CUDA(cudaEventRecord(g_ring.epoch, st));
  g_ring.have_epoch = true;
  g_ring.used = 0;
  g_ring.dropped = 0;
  return KNJ_OK;
}

// Returns a span handle >= 0, or -1 when nothing is recorded (off, no epoch, capturing, ring full).
int knj_span_begin(const char *name, knj_stream_t s) {
  if (!g_ring.on || !g_ring.have_epoch || !name) return -1;
  cudaStream_t st = as_stream(s);
  if (capturing(st)) return -1;
  if (g_ring.used >= (size_t)g_span_capacity) {
    ++g_ring.dropped;
    return -1;
  }
  SpanRec &r = g_ring.recs[g_ring.used];
  size_t n = 0;
  while (name[n] && n + 1 < sizeof(r.name)) { r.name[n] = name[n]; ++n; }
  r.name[n] = 0;
  r.closed = false;
  if (cudaEventRecord(r.a, st) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return (int)g_ring.used++;
}

int knj_span_end(int handle, knj_stream_t s) {
  if (handle < 0) return KNJ_OK;
  KNJ_REQUIRE((size_t)handle < g_ring.used, "knj_span_end: unknown span handle %d", handle);
  KNJ_CUDA(cudaEventRecord(g_ring.recs[handle].b, as_stream(s)));
  g_ring.recs[handle].closed = true;
  return KNJ_OK;
}

uint64_t knj_spans_dropped(void) { return g_ring.dropped; }

// Synchronises on the recorded events and reports every closed span as
// (name, start_ns, end_ns, stream 0, user), offsets from the epoch, in the order recorded.
int knj_spans_flush(void (*cb)(const char *, uint64_t, uint64_t, int, void *), void *user) {
  KNJ_REQUIRE(cb, "knj_spans_flush: null callback");
  if (!g_ring.have_epoch) return KNJ_OK;
  for (size_t i = 0; i < g_ring.used; ++i) {
    SpanRec &r = g_ring.recs[i];
    if (!r.closed) continue;
    KNJ_CUDA(cudaEventSynchronize(r.b));
    float a_ms = 0.f, b_ms = 0.f;
    KNJ_CUDA(cudaEventElapsedTime(&a_ms, g_ring.epoch, r.a));
    KNJ_CUDA(cudaEventElapsedTime(&b_ms, g_ring.epoch, r.b));
    cb(r.name, (uint64_t)((double)a_ms * 1e6 + 0.5), (uint64_t)((double)b_ms * 1e6 + 0.5), 0, user);
  }
  g_ring.used = 0;
  return KNJ_OK;
}

}  // extern "C"
