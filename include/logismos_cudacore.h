/*
 * logismos_cudacore.h - C ABI of the CUDA runtime shim that stands where the reference's
 * `hipcore` crate binds the HIP runtime (crates/hipcore/src/ffi.rs:24, bindgen over
 * crates/hipcore/include/wrapper_runtime.h). Each entry point lists the HIP call site it
 * replaces. Every function returns the raw cudaError_t as u32 (0 = success), the way the
 * reference's `check(code, op)` (crates/hipcore/src/error.rs:222-228) expects a raw status.
 *
 * Conventions kept from hipcore:
 *   - every call makes its device current first (crates/hipcore/src/device.rs:187-193);
 *   - allocation does not zero memory, zero filling is explicit (src/memory.rs:163-182);
 *   - streams are created non-blocking (src/stream.rs:38);
 *   - nothing here panics or aborts; a failing free/destroy reports its status and leaves
 *     the object leaked, as the reference's Drop impls do (src/memory.rs:420-452).
 */
#ifndef LOGISMOS_CUDACORE_H
#define LOGISMOS_CUDACORE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* DeviceProps of crates/hipcore/src/device.rs:36-80, filled from cudaDeviceProp.
 * isa is "sm_100"-style text (the reference stores gcnArchName, e.g. "gfx1100");
 * wavefront_size is the warp size (32). */
typedef struct lg_device_props {
  char isa[32];
  char name[256];
  uint64_t total_vram_bytes;
  int32_t compute_units;
  int32_t wavefront_size;
  int32_t max_threads_per_block;
  uint64_t max_shared_mem_per_block;
  int32_t clock_rate_khz;
  int32_t pci_bus_id;
} lg_device_props_t;

/* hipGetDeviceCount - src/device.rs:103, :297 */
uint32_t lg_device_count(int32_t* count);
/* hipSetDevice - src/device.rs:110, :190. An out-of-range ordinal fails deterministically
 * (cudaErrorInvalidDevice), which is what Device::invalid_for_test relies on (:125-153). */
uint32_t lg_device_set_current(int32_t ordinal);
/* hipGetDeviceProperties - src/device.rs:117 */
uint32_t lg_device_props_get(int32_t ordinal, lg_device_props_t* out);
/* hipMemGetInfo - src/device.rs:206 */
uint32_t lg_device_mem_info(int32_t ordinal, uint64_t* free_bytes, uint64_t* total_bytes);
/* hipDeviceSynchronize - src/device.rs:225 */
uint32_t lg_device_synchronize(int32_t ordinal);

/* hipMalloc - src/memory.rs:63 */
uint32_t lg_malloc(int32_t ordinal, size_t bytes, void** dev_ptr);
/* hipFree - src/memory.rs:440 */
uint32_t lg_free(int32_t ordinal, void* dev_ptr);
/* hipMemset - src/memory.rs:179 */
uint32_t lg_memset(int32_t ordinal, void* dev_ptr, int32_t value, size_t bytes);
/* hipMemcpy(HostToDevice) - src/memory.rs:152 */
uint32_t lg_memcpy_h2d(int32_t ordinal, void* dev_dst, const void* host_src, size_t bytes);
/* hipMemcpy(DeviceToHost) - src/memory.rs:205 */
uint32_t lg_memcpy_d2h(int32_t ordinal, void* host_dst, const void* dev_src, size_t bytes);
/* hipMemcpyAsync(HostToDevice) - src/memory.rs:274. The caller keeps both buffers alive and
 * untouched until the stream is synchronised (PendingCopy, src/memory.rs:306-418). */
uint32_t lg_memcpy_h2d_async(int32_t ordinal, void* dev_dst, const void* host_src, size_t bytes,
                             void* stream);

/* hipStreamCreateWithFlags(hipStreamNonBlocking) - src/stream.rs:38 */
uint32_t lg_stream_create(int32_t ordinal, void** stream);
/* hipStreamSynchronize - src/stream.rs:81 (stream may be NULL = the null stream, :51) */
uint32_t lg_stream_synchronize(int32_t ordinal, void* stream);
/* hipStreamDestroy - src/stream.rs:123 */
uint32_t lg_stream_destroy(int32_t ordinal, void* stream);
/* hipEventCreate - src/stream.rs:163 */
uint32_t lg_event_create(int32_t ordinal, void** event);
/* hipEventRecord - src/stream.rs:95 */
uint32_t lg_event_record(int32_t ordinal, void* event, void* stream);
/* hipEventSynchronize - src/stream.rs:181 */
uint32_t lg_event_synchronize(int32_t ordinal, void* event);
/* hipEventElapsedTime - src/stream.rs:196 */
uint32_t lg_event_elapsed_ms(void* start, void* end, float* ms);
/* hipEventDestroy - src/stream.rs:239 */
uint32_t lg_event_destroy(int32_t ordinal, void* event);

/* ErrorKind::from_raw (src/error.rs:126-147), re-derived for cudaError_t numbering:
 * HIP's 719/700/701/702/53/500/600/35 are not CUDA's. Kinds, in the reference's order: */
enum lg_error_kind {
  LG_ERR_NONE = 0,
  LG_ERR_INVALID_VALUE,
  LG_ERR_OUT_OF_MEMORY,
  LG_ERR_NOT_INITIALIZED,
  LG_ERR_DEINITIALIZED,
  LG_ERR_INSUFFICIENT_DRIVER,
  LG_ERR_PRIOR_LAUNCH_FAILURE,
  LG_ERR_LAUNCH_OUT_OF_RESOURCES,
  LG_ERR_LAUNCH_TIMEOUT,
  LG_ERR_LAUNCH_FAILURE,
  LG_ERR_NOT_FOUND,
  LG_ERR_NOT_READY,
  LG_ERR_ILLEGAL_ADDRESS,
  LG_ERR_UNKNOWN
};
uint32_t lg_error_kind_from_raw(uint32_t code);
const char* lg_error_kind_name(uint32_t kind);
/* cudaGetErrorString, for messages */
const char* lg_error_string(uint32_t code);

#ifdef __cplusplus
}
#endif
#endif
