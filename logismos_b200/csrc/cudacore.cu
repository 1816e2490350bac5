// CUDA runtime shim behind include/logismos_cudacore.h: the surface the reference's hipcore
// crate takes from the HIP runtime, expressed over the CUDA runtime.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

#include "logismos_cudacore.h"

namespace {
// Every entry point returns its status explicitly, so a failure must not also stay behind in the
// runtime's "last error" slot, where the next kernel launch of the process would pick it up.
inline uint32_t done(cudaError_t e) {
  if (e != cudaSuccess) (void)cudaGetLastError();
  return (uint32_t)e;
}
inline uint32_t make_current(int32_t ordinal) { return done(cudaSetDevice(ordinal)); }
}  // namespace

#define LG_CURRENT(ord)                          \
  do {                                           \
    uint32_t rc_ = make_current(ord);            \
    if (rc_ != 0) return rc_;                    \
  } while (0)

extern "C" {

uint32_t lg_device_count(int32_t* count) {
  int c = 0;
  cudaError_t e = cudaGetDeviceCount(&c);
  if (count) *count = (e == cudaSuccess) ? c : 0;
  return done(e);
}

uint32_t lg_device_set_current(int32_t ordinal) { return make_current(ordinal); }

uint32_t lg_device_props_get(int32_t ordinal, lg_device_props_t* out) {
  if (!out) return (uint32_t)cudaErrorInvalidValue;
  cudaDeviceProp p;
  cudaError_t e = cudaGetDeviceProperties(&p, ordinal);
  if (e != cudaSuccess) return done(e);
  std::memset(out, 0, sizeof(*out));
  std::snprintf(out->isa, sizeof(out->isa), "sm_%d%d", p.major, p.minor);
  std::snprintf(out->name, sizeof(out->name), "%s", p.name);
  out->total_vram_bytes = (uint64_t)p.totalGlobalMem;
  out->compute_units = p.multiProcessorCount;
  out->wavefront_size = p.warpSize;
  out->max_threads_per_block = p.maxThreadsPerBlock;
  out->max_shared_mem_per_block = (uint64_t)p.sharedMemPerBlockOptin;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ordinal);
  out->clock_rate_khz = khz;
  out->pci_bus_id = p.pciBusID;
  return 0;
}

uint32_t lg_device_mem_info(int32_t ordinal, uint64_t* free_bytes, uint64_t* total_bytes) {
  LG_CURRENT(ordinal);
  size_t f = 0, t = 0;
  cudaError_t e = cudaMemGetInfo(&f, &t);
  if (free_bytes) *free_bytes = f;
  if (total_bytes) *total_bytes = t;
  return done(e);
}

uint32_t lg_device_synchronize(int32_t ordinal) {
  LG_CURRENT(ordinal);
  return done(cudaDeviceSynchronize());
}

uint32_t lg_malloc(int32_t ordinal, size_t bytes, void** dev_ptr) {
  if (!dev_ptr) return (uint32_t)cudaErrorInvalidValue;
  *dev_ptr = nullptr;
  LG_CURRENT(ordinal);
  return done(cudaMalloc(dev_ptr, bytes));
}

uint32_t lg_free(int32_t ordinal, void* dev_ptr) {
  LG_CURRENT(ordinal);
  return done(cudaFree(dev_ptr));
}

uint32_t lg_memset(int32_t ordinal, void* dev_ptr, int32_t value, size_t bytes) {
  LG_CURRENT(ordinal);
  return done(cudaMemset(dev_ptr, value, bytes));
}

uint32_t lg_memcpy_h2d(int32_t ordinal, void* dev_dst, const void* host_src, size_t bytes) {
  LG_CURRENT(ordinal);
  return done(cudaMemcpy(dev_dst, host_src, bytes, cudaMemcpyHostToDevice));
}

uint32_t lg_memcpy_d2h(int32_t ordinal, void* host_dst, const void* dev_src, size_t bytes) {
  LG_CURRENT(ordinal);
  return done(cudaMemcpy(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost));
}

uint32_t lg_memcpy_h2d_async(int32_t ordinal, void* dev_dst, const void* host_src, size_t bytes,
                             void* stream) {
  LG_CURRENT(ordinal);
  return done(cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice,
                                   (cudaStream_t)stream));
}

uint32_t lg_stream_create(int32_t ordinal, void** stream) {
  if (!stream) return (uint32_t)cudaErrorInvalidValue;
  *stream = nullptr;
  LG_CURRENT(ordinal);
  cudaStream_t s;
  cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  if (e == cudaSuccess) *stream = (void*)s;
  return done(e);
}

uint32_t lg_stream_synchronize(int32_t ordinal, void* stream) {
  LG_CURRENT(ordinal);
  return done(cudaStreamSynchronize((cudaStream_t)stream));
}

uint32_t lg_stream_destroy(int32_t ordinal, void* stream) {
  LG_CURRENT(ordinal);
  return done(cudaStreamDestroy((cudaStream_t)stream));
}

uint32_t lg_event_create(int32_t ordinal, void** event) {
  if (!event) return (uint32_t)cudaErrorInvalidValue;
  *event = nullptr;
  LG_CURRENT(ordinal);
  cudaEvent_t ev;
  cudaError_t e = cudaEventCreate(&ev);
  if (e == cudaSuccess) *event = (void*)ev;
  return done(e);
}

uint32_t lg_event_record(int32_t ordinal, void* event, void* stream) {
  LG_CURRENT(ordinal);
  return done(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
}

uint32_t lg_event_synchronize(int32_t ordinal, void* event) {
  LG_CURRENT(ordinal);
  return done(cudaEventSynchronize((cudaEvent_t)event));
}

uint32_t lg_event_elapsed_ms(void* start, void* end, float* ms) {
  if (!ms) return (uint32_t)cudaErrorInvalidValue;
  return done(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)end));
}

uint32_t lg_event_destroy(int32_t ordinal, void* event) {
  LG_CURRENT(ordinal);
  return done(cudaEventDestroy((cudaEvent_t)event));
}

uint32_t lg_error_kind_from_raw(uint32_t code) {
  switch ((cudaError_t)code) {
    case cudaSuccess: return LG_ERR_NONE;
    case cudaErrorInvalidValue: return LG_ERR_INVALID_VALUE;
    case cudaErrorMemoryAllocation: return LG_ERR_OUT_OF_MEMORY;
    case cudaErrorInitializationError: return LG_ERR_NOT_INITIALIZED;
    case cudaErrorCudartUnloading: return LG_ERR_DEINITIALIZED;
    case cudaErrorInsufficientDriver: return LG_ERR_INSUFFICIENT_DRIVER;
    case cudaErrorLaunchOutOfResources: return LG_ERR_LAUNCH_OUT_OF_RESOURCES;
    case cudaErrorLaunchTimeout: return LG_ERR_LAUNCH_TIMEOUT;
    case cudaErrorLaunchFailure: return LG_ERR_LAUNCH_FAILURE;
    case cudaErrorSymbolNotFound: return LG_ERR_NOT_FOUND;
    case cudaErrorNotReady: return LG_ERR_NOT_READY;
    case cudaErrorIllegalAddress: return LG_ERR_ILLEGAL_ADDRESS;
    default: break;
  }
  // hipErrorPriorLaunchFailure has no CUDA twin with its own number; CUDA reports a sticky
  // context error by repeating the original code, which the cases above already classify.
  return LG_ERR_UNKNOWN;
}

}  // extern "C"

#include <atomic>
#include <cstdlib>
namespace lg {
static std::atomic<int> g_deterministic{-1};
bool deterministic() {
  int v = g_deterministic.load(std::memory_order_relaxed);
  if (v < 0) {  // first use: the environment decides unless the host has set it
    const char* e = std::getenv("LOGISMOS_DETERMINISTIC");
    v = (e && e[0] && e[0] != '0') ? 1 : 0;
    g_deterministic.store(v, std::memory_order_relaxed);
  }
  return v != 0;
}
static std::atomic<int> g_dependent_launch{-1};
bool dependent_launch() {
  int v = g_dependent_launch.load(std::memory_order_relaxed);
  if (v < 0) {  // first use: on unless the environment says 0
    const char* e = std::getenv("LOGISMOS_DEPENDENT_LAUNCH");
    v = (e && e[0] == '0') ? 0 : 1;
    g_dependent_launch.store(v, std::memory_order_relaxed);
  }
  return v != 0;
}
}  // namespace lg

extern "C" {

void logismos_set_dependent_launch(int32_t on) { lg::g_dependent_launch.store(on ? 1 : 0, std::memory_order_relaxed); }
int32_t logismos_get_dependent_launch(void) { return lg::dependent_launch() ? 1 : 0; }
void logismos_set_deterministic(int32_t on) { lg::g_deterministic.store(on ? 1 : 0, std::memory_order_relaxed); }
int32_t logismos_get_deterministic(void) { return lg::deterministic() ? 1 : 0; }

const char* lg_error_kind_name(uint32_t kind) {
  static const char* names[] = {"None", "InvalidValue", "OutOfMemory", "NotInitialized",
                                "Deinitialized", "InsufficientDriver", "PriorLaunchFailure",
                                "LaunchOutOfResources", "LaunchTimeout", "LaunchFailure",
                                "NotFound", "NotReady", "IllegalAddress", "Unknown"};
  return kind <= LG_ERR_UNKNOWN ? names[kind] : "Unknown";
}

const char* lg_error_string(uint32_t code) { return cudaGetErrorString((cudaError_t)code); }

}  // extern "C"
