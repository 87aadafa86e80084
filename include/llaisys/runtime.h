/*
 * llaisys C ABI -- per-device runtime table.
 *
 * The table is twelve function pointers in a fixed order (reference:
 * include/llaisys/runtime.h:25-38); the reference's Python frontend mirrors the
 * struct field by field and calls the pointers directly with raw addresses
 * (reference: python/llaisys/libllaisys/runtime.py:24-38, python/llaisys/runtime.py:12-68),
 * so neither the order nor any signature may change.
 *
 * NVIDIA semantics in this library: streams are blocking CUDA streams, so a
 * memcpy_sync (issued on the legacy default stream) is ordered after every
 * operator already queued on a runtime stream -- callers read results straight
 * after an op without an explicit synchronise, as the reference's tests do
 * (reference: test/test_utils.py:143-149).
 */
#ifndef LLAISYS_RUNTIME_H
#define LLAISYS_RUNTIME_H

#include "../llaisys.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef int (*get_device_count_api)(void);
typedef void (*set_device_api)(int);
typedef void (*device_synchronize_api)(void);
typedef llaisysStream_t (*create_stream_api)(void);
typedef void (*destroy_stream_api)(llaisysStream_t);
typedef void (*stream_synchronize_api)(llaisysStream_t);
typedef void *(*malloc_device_api)(size_t);
typedef void (*free_device_api)(void *);
typedef void *(*malloc_host_api)(size_t);
typedef void (*free_host_api)(void *);
typedef void (*memcpy_sync_api)(void *, const void *, size_t, llaisysMemcpyKind_t);
typedef void (*memcpy_async_api)(void *, const void *, size_t, llaisysMemcpyKind_t, llaisysStream_t);

typedef struct LlaisysRuntimeAPI {
    get_device_count_api get_device_count;
    set_device_api set_device;
    device_synchronize_api device_synchronize;
    create_stream_api create_stream;
    destroy_stream_api destroy_stream;
    stream_synchronize_api stream_synchronize;
    malloc_device_api malloc_device;
    free_device_api free_device;
    malloc_host_api malloc_host;
    free_host_api free_host;
    memcpy_sync_api memcpy_sync;
    memcpy_async_api memcpy_async;
} LlaisysRuntimeAPI;

/* Table for a device type. A device type this build cannot drive reports
 * get_device_count() == 0 and throws from everything else
 * (reference: src/device/runtime_api.cpp:5-71). */
LLAISYS_API const LlaisysRuntimeAPI *llaisysGetRuntimeAPI(llaisysDeviceType_t device_type);

/* Makes (device_type, device_id) current for the calling host thread
 * (reference: include/llaisys/runtime.h:44, src/llaisys/runtime.cc:6-8). */
LLAISYS_API void llaisysSetContextRuntime(llaisysDeviceType_t device_type, int device_id);

/* NEW (no counterpart in the reference): the stream on which the calling thread's
 * current runtime queues operators, so a caller can record events on it or wrap it
 * in its own framework's stream object. NULL on CPU. */
LLAISYS_API llaisysStream_t llaisysGetContextStream(void);

#ifdef __cplusplus
}
#endif

#endif /* LLAISYS_RUNTIME_H */
