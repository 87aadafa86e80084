#include "runtime_api.hpp"

#include "../common/check.hpp"

#include <cstdlib>
#include <cstring>

namespace llaisys::device {

// ---- a device type that is compiled out -------------------------------------------------------
namespace absent {
int count() { return 0; }
void set(int) { EXCEPTION_UNSUPPORTED_DEVICE; }
void sync() { EXCEPTION_UNSUPPORTED_DEVICE; }
llaisysStream_t stream_new() { EXCEPTION_UNSUPPORTED_DEVICE; }
void stream_op(llaisysStream_t) { EXCEPTION_UNSUPPORTED_DEVICE; }
void *alloc(size_t) { EXCEPTION_UNSUPPORTED_DEVICE; }
void release(void *) { EXCEPTION_UNSUPPORTED_DEVICE; }
void copy(void *, const void *, size_t, llaisysMemcpyKind_t) { EXCEPTION_UNSUPPORTED_DEVICE; }
void copy_async(void *, const void *, size_t, llaisysMemcpyKind_t, llaisysStream_t) { EXCEPTION_UNSUPPORTED_DEVICE; }

const LlaisysRuntimeAPI table = {count, set,     sync,  stream_new, stream_op, stream_op,
                                 alloc, release, alloc, release,    copy,      copy_async};
} // namespace absent

// ---- the host itself as a device (reference: src/device/cpu/cpu_runtime_api.cpp:9-68) ------------
namespace host {
int count() { return 1; }
void set(int) {}
void sync() {}
llaisysStream_t stream_new() { return nullptr; }
void stream_op(llaisysStream_t) {}
void *alloc(size_t bytes) { return std::malloc(bytes ? bytes : 1); }
void release(void *p) { std::free(p); }
void copy(void *dst, const void *src, size_t bytes, llaisysMemcpyKind_t) { std::memcpy(dst, src, bytes); }
void copy_async(void *dst, const void *src, size_t bytes, llaisysMemcpyKind_t kind, llaisysStream_t) {
    copy(dst, src, bytes, kind);
}

const LlaisysRuntimeAPI table = {count, set,     sync,  stream_new, stream_op, stream_op,
                                 alloc, release, alloc, release,    copy,      copy_async};
} // namespace host

const LlaisysRuntimeAPI *getUnsupportedRuntimeAPI() { return &absent::table; }

namespace cpu {
const LlaisysRuntimeAPI *getRuntimeAPI() { return &host::table; }
} // namespace cpu

const LlaisysRuntimeAPI *getRuntimeAPI(llaisysDeviceType_t device_type) {
    switch (device_type) {
    case LLAISYS_DEVICE_CPU:
        return cpu::getRuntimeAPI();
    case LLAISYS_DEVICE_NVIDIA:
#ifdef ENABLE_NVIDIA_API
        return nvidia::getRuntimeAPI();
#else
        return getUnsupportedRuntimeAPI();
#endif
    default:
        EXCEPTION_UNSUPPORTED_DEVICE;
    }
}

} // namespace llaisys::device
