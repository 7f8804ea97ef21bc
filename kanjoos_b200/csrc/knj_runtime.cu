// knj_runtime.cu -- the device layer of the C-ABI: a thin, stateless cover over
// the CUDA runtime for the calls the reference's drivers make on HIP
// (include/knj_device.h lists the HIP call each function stands for).
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "knj_common.cuh"

namespace knj {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return KNJ_E_RUNTIME;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int make_row_tensor_map(CUtensorMap *map, const void *base, uint64_t rows, uint32_t row_bytes, uint32_t box_bytes,
                        uint32_t box_rows) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || !fn) {
      set_error("cuTensorMapEncodeTiled is not available from this driver");
      return KNJ_E_RUNTIME;
    }
    encode = reinterpret_cast<EncodeFn>(fn);
  }
  KNJ_REQUIRE(row_bytes % 16 == 0 && box_bytes % 16 == 0 && box_bytes <= 1024 && box_rows >= 1 && box_rows <= 256 &&
                  aligned16(base),
              "tensor map: rows of %u bytes / boxes of %u x %u bytes are not TMA-addressable", row_bytes, box_rows, box_bytes);
  const cuuint64_t dims[2] = {row_bytes / 4, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_bytes / 4, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with driver status %d", (int)r);
    return KNJ_E_RUNTIME;
  }
  return KNJ_OK;
}

}  // namespace knj

using namespace knj;

namespace knj {
int g_chain_overlap = 1;
}

extern "C" {

// 1 (default): the kernels of a decode layer are launched with programmatic stream serialization, so each
// grid is scheduled while its predecessor drains; 0: plain launches.
void knj_launch_overlap(int on) { g_chain_overlap = on ? 1 : 0; }


const char *knj_last_error_string(void) { return g_err; }

int knj_dev_count(int *n) {
  KNJ_REQUIRE(n, "knj_dev_count: null out pointer");
  cudaError_t e = cudaGetDeviceCount(n);
  if (e != cudaSuccess) {
    *n = 0;
    return cuda_fail(e, "cudaGetDeviceCount");
  }
  return KNJ_OK;
}

int knj_dev_open(int idx) {
  int n = 0;
  int rc = knj_dev_count(&n);
  if (rc) return rc;
  KNJ_REQUIRE(idx >= 0 && idx < n, "knj_dev_open: device %d of %d", idx, n);
  int major = 0;
  KNJ_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, idx));
  if (major != 10) {
    set_error("knj_dev_open: device %d has compute capability %d.x; this library is built for sm_100a only", idx,
              major);
    return KNJ_E_ARCH;
  }
  KNJ_CUDA(cudaSetDevice(idx));
  return KNJ_OK;
}

int knj_dev_current(int *idx) {
  KNJ_REQUIRE(idx, "knj_dev_current: null out pointer");
  KNJ_CUDA(cudaGetDevice(idx));
  return KNJ_OK;
}

int knj_dev_caps(int idx, knj_device_caps *out) {
  KNJ_REQUIRE(out, "knj_dev_caps: null out pointer");
  memset(out, 0, sizeof *out);
  cudaDeviceProp p;
  KNJ_CUDA(cudaGetDeviceProperties(&p, idx));
  snprintf(out->arch, sizeof out->arch, "sm_%d%d", p.major, p.minor);
  snprintf(out->name, sizeof out->name, "%s", p.name);
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->has_mma = p.major == 10;
  out->has_fp8 = p.major >= 9;
  out->has_dot_builtin = 0;
  out->wave_size = p.warpSize;
  out->vram_total = p.totalGlobalMem;
  int cur = -1;
  cudaGetDevice(&cur);
  if (cur == idx) {
    size_t fr = 0, tot = 0;
    if (cudaMemGetInfo(&fr, &tot) == cudaSuccess) out->vram_usable = fr;
  }
  out->rebar_full_aperture = 1;  // the whole of HBM is mapped; there is no aperture window on this platform
  out->sms = (uint32_t)p.multiProcessorCount;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, idx);
  out->clock_khz = (uint32_t)khz;
  out->max_streams = 128;  // hardware work queues are not a bound the runtime exposes; connections default
  out->num_queue_groups = (uint32_t)p.asyncEngineCount;
  out->smem_per_block_optin = (uint32_t)p.sharedMemPerBlockOptin;
  out->l2_bytes = (uint32_t)p.l2CacheSize;
  return KNJ_OK;
}

int knj_dev_sync(void) {
  KNJ_CUDA(cudaDeviceSynchronize());
  return KNJ_OK;
}

int knj_mem_info(size_t *free_bytes, size_t *total) {
  KNJ_REQUIRE(free_bytes && total, "knj_mem_info: null out pointer");
  KNJ_CUDA(cudaMemGetInfo(free_bytes, total));
  return KNJ_OK;
}

int knj_arch_check(void) {
  const char *env = getenv("KNJ_BUILD_ARCH");
  if (!env || !*env) {
    set_error("KNJ_BUILD_ARCH is not set: refusing to touch the device");
    return KNJ_EXIT_REFUSED;
  }
  if (strcmp(env, "sm_100") != 0) {
    set_error("DECLINED: KNJ_BUILD_ARCH=%s, library is built for sm_100", env);
    return KNJ_EXIT_DECLINED;
  }
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    set_error("no CUDA device");
    return KNJ_EXIT_RUNTIME;
  }
  int dev = 0, major = 0, minor = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  if (major != 10) {
    set_error("DECLINED: built for sm_100, attached device is sm_%d%d. This is a skip, not a result.", major, minor);
    return KNJ_EXIT_DECLINED;
  }
  return KNJ_EXIT_PASS;
}

int knj_malloc(void **p, size_t bytes) {
  KNJ_REQUIRE(p, "knj_malloc: null out pointer");
  KNJ_CUDA(cudaMalloc(p, bytes));
  return KNJ_OK;
}
int knj_free(void *p) {
  KNJ_CUDA(cudaFree(p));
  return KNJ_OK;
}
int knj_host_malloc(void **p, size_t bytes) {
  KNJ_REQUIRE(p, "knj_host_malloc: null out pointer");
  KNJ_CUDA(cudaMallocHost(p, bytes));
  return KNJ_OK;
}
int knj_host_free(void *p) {
  KNJ_CUDA(cudaFreeHost(p));
  return KNJ_OK;
}
int knj_memset(void *p, int byte, size_t n, knj_stream_t s) {
  KNJ_CUDA(cudaMemsetAsync(p, byte, n, as_stream(s)));
  return KNJ_OK;
}
int knj_memcpy_h2d(void *dst, const void *src, size_t n) {
  KNJ_CUDA(cudaMemcpy(dst, src, n, cudaMemcpyHostToDevice));
  return KNJ_OK;
}
int knj_memcpy_d2h(void *dst, const void *src, size_t n) {
  KNJ_CUDA(cudaMemcpy(dst, src, n, cudaMemcpyDeviceToHost));
  return KNJ_OK;
}
int knj_memcpy_d2d(void *dst, const void *src, size_t n) {
  KNJ_CUDA(cudaMemcpy(dst, src, n, cudaMemcpyDeviceToDevice));
  return KNJ_OK;
}
int knj_memcpy_h2d_async(void *dst, const void *src, size_t n, knj_stream_t s) {
  KNJ_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, as_stream(s)));
  return KNJ_OK;
}
int knj_memcpy_d2h_async(void *dst, const void *src, size_t n, knj_stream_t s) {
  KNJ_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, as_stream(s)));
  return KNJ_OK;
}
int knj_memcpy_d2d_async(void *dst, const void *src, size_t n, knj_stream_t s) {
  KNJ_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, as_stream(s)));
  return KNJ_OK;
}

int knj_stream_create(knj_stream_t *s) {
  KNJ_REQUIRE(s, "knj_stream_create: null out pointer");
  cudaStream_t st;
  KNJ_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  *s = st;
  return KNJ_OK;
}
int knj_stream_destroy(knj_stream_t s) {
  KNJ_CUDA(cudaStreamDestroy(as_stream(s)));
  return KNJ_OK;
}
int knj_stream_sync(knj_stream_t s) {
  KNJ_CUDA(cudaStreamSynchronize(as_stream(s)));
  return KNJ_OK;
}
int knj_stream_query(knj_stream_t s) {
  cudaError_t e = cudaStreamQuery(as_stream(s));
  if (e == cudaErrorNotReady) return KNJ_E_NOTREADY;
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamQuery");
  return KNJ_OK;
}
int knj_stream_wait_event(knj_stream_t s, knj_event_t e) {
  KNJ_CUDA(cudaStreamWaitEvent(as_stream(s), reinterpret_cast<cudaEvent_t>(e), 0));
  return KNJ_OK;
}
int knj_event_create(knj_event_t *e, int timing) {
  KNJ_REQUIRE(e, "knj_event_create: null out pointer");
  cudaEvent_t ev;
  KNJ_CUDA(cudaEventCreateWithFlags(&ev, timing ? cudaEventDefault : cudaEventDisableTiming));
  *e = ev;
  return KNJ_OK;
}
int knj_event_destroy(knj_event_t e) {
  KNJ_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(e)));
  return KNJ_OK;
}
int knj_event_record(knj_event_t e, knj_stream_t s) {
  KNJ_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(e), as_stream(s)));
  return KNJ_OK;
}
int knj_event_query(knj_event_t e) {
  cudaError_t r = cudaEventQuery(reinterpret_cast<cudaEvent_t>(e));
  if (r == cudaErrorNotReady) return KNJ_E_NOTREADY;
  if (r != cudaSuccess) return cuda_fail(r, "cudaEventQuery");
  return KNJ_OK;
}
int knj_event_sync(knj_event_t e) {
  KNJ_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(e)));
  return KNJ_OK;
}
int knj_event_elapsed_ms(float *ms, knj_event_t a, knj_event_t b) {
  KNJ_REQUIRE(ms, "knj_event_elapsed_ms: null out pointer");
  KNJ_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(a), reinterpret_cast<cudaEvent_t>(b)));
  return KNJ_OK;
}

int knj_graph_begin(knj_stream_t s) {
  KNJ_CUDA(cudaStreamBeginCapture(as_stream(s), cudaStreamCaptureModeThreadLocal));
  return KNJ_OK;
}
int knj_graph_end(knj_stream_t s, knj_graph_t *g) {
  KNJ_REQUIRE(g, "knj_graph_end: null out pointer");
  cudaGraph_t graph = nullptr;
  KNJ_CUDA(cudaStreamEndCapture(as_stream(s), &graph));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
  *g = exec;
  return KNJ_OK;
}
int knj_graph_launch(knj_graph_t g, knj_stream_t s) {
  KNJ_CUDA(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(g), as_stream(s)));
  return KNJ_OK;
}
int knj_graph_destroy(knj_graph_t g) {
  KNJ_CUDA(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(g)));
  return KNJ_OK;
}

}  // extern "C"
