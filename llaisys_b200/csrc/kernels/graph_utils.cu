// Small runtime helpers for the model's device-resident decode loop: CUDA graph capture / replay, event timing, and
// the kernel that carries the loop state from one step to the next without a host round trip.
#include "device_utils.cuh"
#include "kernels.hpp"

#include <cuda.h>

namespace llaisys::kernels {

namespace {

// After a greedy step: feed the chosen tokens back as the next inputs, log them, advance positions and lengths.
__global__ void advance_decode_state_kernel(int64_t *__restrict__ tokens, const int64_t *__restrict__ next,
                                            int64_t *__restrict__ pos64, int32_t *__restrict__ pos32,
                                            int32_t *__restrict__ kv_lens, int64_t *__restrict__ log,
                                            int32_t *__restrict__ step_counter, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int step = *step_counter;
    if (i < n) {
        const int64_t t = next[i];
        tokens[i] = t;
        log[int64_t(step) * n + i] = t;
        pos64[i] += 1;
        pos32[i] += 1;
        kv_lens[i] += 1;
    }
}

// The step counter is bumped by its own launch, after every block of the kernel above has read it.
__global__ void bump_counter_kernel(int32_t *counter) { *counter += 1; }

} // namespace

void advance_decode_state(stream_t stream, int64_t *tokens, const int64_t *next, int64_t *pos64, int32_t *pos32,
                          int32_t *kv_lens, int64_t *log, int32_t *step_counter, int n) {
    auto s = static_cast<cudaStream_t>(stream);
    advance_decode_state_kernel<<<(n + 255) / 256, 256, 0, s>>>(tokens, next, pos64, pos32, kv_lens, log, step_counter, n);
    bump_counter_kernel<<<1, 1, 0, s>>>(step_counter);
    check_launch("advance_decode_state");
}

const void *mapped_host_alias(const void *host_ptr, size_t bytes) {
    cudaPointerAttributes first;
    if (host_ptr == nullptr || bytes == 0 || cudaPointerGetAttributes(&first, host_ptr) != cudaSuccess ||
        first.type != cudaMemoryTypeHost || first.devicePointer == nullptr) {
        (void)cudaGetLastError();
        return nullptr;
    }
    // The whole buffer must lie in ONE mapped allocation: a buffer that starts in a page-locked block and runs past its
    // end would have the kernel read or write whatever lies behind it.
    using RangeFn = CUresult (*)(CUdeviceptr *, size_t *, CUdeviceptr);
    static const RangeFn range = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &res) != cudaSuccess ||
            res != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            return RangeFn(nullptr);
        }
        return reinterpret_cast<RangeFn>(sym);
    }();
    if (range == nullptr) {
        return nullptr;
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    const CUdeviceptr dptr = reinterpret_cast<CUdeviceptr>(first.devicePointer);
    if (range(&base, &size, dptr) != CUDA_SUCCESS || dptr < base || dptr - base + bytes > size) {
        return nullptr;
    }
    return first.devicePointer;
}

void graph_capture_begin(stream_t stream) {
    LLAISYS_CUDA_CHECK(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal));
}

void *graph_capture_end(stream_t stream) {
    cudaGraph_t graph = nullptr;
    LLAISYS_CUDA_CHECK(cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &graph));
    cudaGraphExec_t exec = nullptr;
    const cudaError_t err = cudaGraphInstantiate(&exec, graph, 0);
    (void)cudaGraphDestroy(graph);
    LLAISYS_CUDA_CHECK(err);
    return exec;
}

void graph_launch(void *exec, stream_t stream) {
    LLAISYS_CUDA_CHECK(cudaGraphLaunch(static_cast<cudaGraphExec_t>(exec), static_cast<cudaStream_t>(stream)));
}

void graph_destroy(void *exec) {
    if (exec != nullptr) {
        (void)cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(exec));
    }
}

void *event_create() {
    cudaEvent_t e = nullptr;
    LLAISYS_CUDA_CHECK(cudaEventCreate(&e));
    return e;
}
void event_record(void *event, stream_t stream) {
    LLAISYS_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
}
float event_elapsed_ms(void *start, void *stop) {
    LLAISYS_CUDA_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)));
    float ms = 0.f;
    LLAISYS_CUDA_CHECK(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
    return ms;
}
void event_destroy(void *event) {
    if (event != nullptr) {
        (void)cudaEventDestroy(static_cast<cudaEvent_t>(event));
    }
}

} // namespace llaisys::kernels
