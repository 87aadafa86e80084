// CUDA implementation of the runtime table (the reference ships twelve stubs here:
// src/device/nvidia/nvidia_runtime_api.cu:9-54, and its memcpyAsync stub even lacks the stream
// parameter, :52).
//
// Ordering model: runtime streams are BLOCKING streams and memcpy_sync goes through the legacy
// default stream, which waits for all blocking streams of the context. An operator queued on a
// runtime stream is therefore complete before a following memcpy_sync reads its output, and work a
// caller queued on the legacy default stream (PyTorch's default) is complete before a following
// operator starts. That is what lets the reference's tests copy results out right after an
// operator call with no synchronise in between (test/test_utils.py:143-149).
#include "runtime_api.hpp"

#include "../common/check.hpp"
#include "cuda_check.cuh"

#include <cuda_runtime.h>

namespace llaisys::device::nvidia {

namespace {

int count() {
    int n = 0;
    // No driver / no GPU is not an error for a probe: report zero devices.
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

void set(int device) { LLAISYS_CUDA_CHECK(cudaSetDevice(device)); }
void sync() { LLAISYS_CUDA_CHECK(cudaDeviceSynchronize()); }

llaisysStream_t stream_new() {
    cudaStream_t s = nullptr;
    LLAISYS_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamDefault));
    return static_cast<llaisysStream_t>(s);
}
// Releases never throw: they also run from thread-exit and process-exit destructors, where the CUDA
// runtime may already be unloading and reports that as an error.
void stream_free(llaisysStream_t s) {
    if (cudaStreamDestroy(static_cast<cudaStream_t>(s)) != cudaSuccess) {
        (void)cudaGetLastError();
    }
}
void stream_sync(llaisysStream_t s) { LLAISYS_CUDA_CHECK(cudaStreamSynchronize(static_cast<cudaStream_t>(s))); }

void *dev_alloc(size_t bytes) {
    void *p = nullptr;
    LLAISYS_CUDA_CHECK(cudaMalloc(&p, bytes ? bytes : 1));
    return p;
}
void dev_free(void *p) {
    if (cudaFree(p) != cudaSuccess) {
        (void)cudaGetLastError();
    }
}

void *pinned_alloc(size_t bytes) {
    void *p = nullptr;
    LLAISYS_CUDA_CHECK(cudaMallocHost(&p, bytes ? bytes : 1));
    return p;
}
void pinned_free(void *p) {
    if (cudaFreeHost(p) != cudaSuccess) {
        (void)cudaGetLastError();
    }
}

cudaMemcpyKind to_cuda(llaisysMemcpyKind_t kind) {
    switch (kind) {
    case LLAISYS_MEMCPY_H2H:
        return cudaMemcpyHostToHost;
    case LLAISYS_MEMCPY_H2D:
        return cudaMemcpyHostToDevice;
    case LLAISYS_MEMCPY_D2H:
        return cudaMemcpyDeviceToHost;
    case LLAISYS_MEMCPY_D2D:
        return cudaMemcpyDeviceToDevice;
    }
    CHECK_ARGUMENT(false, "unknown memcpy kind");
    return cudaMemcpyDefault;
}

void copy(void *dst, const void *src, size_t bytes, llaisysMemcpyKind_t kind) {
    if (bytes == 0) {
        return;
    }
    LLAISYS_CUDA_CHECK(cudaMemcpy(dst, src, bytes, to_cuda(kind)));
}

void copy_async(void *dst, const void *src, size_t bytes, llaisysMemcpyKind_t kind, llaisysStream_t stream) {
    if (bytes == 0) {
        return;
    }
    LLAISYS_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, to_cuda(kind), static_cast<cudaStream_t>(stream)));
}

const LlaisysRuntimeAPI table = {count,    set,          sync,        stream_new, stream_free, stream_sync,
                                 dev_alloc, dev_free,    pinned_alloc, pinned_free, copy,       copy_async};

} // namespace

const LlaisysRuntimeAPI *getRuntimeAPI() { return &table; }

} // namespace llaisys::device::nvidia
