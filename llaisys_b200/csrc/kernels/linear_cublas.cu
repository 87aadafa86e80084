// linear on the device: out[M, N] = in[M, K] . weight[N, K]^T. Decode-sized calls (at most 128 rows, 16-bit) go to the
// hand-written weight-streaming kernel (skinny_gemm_tc.cu); everything else is a plain library GEMM through cuBLAS.
//
// cuBLAS is opened with dlopen at the first call instead of being linked: the library then loads on machines without
// it, and inside a process that already carries a cuBLAS (PyTorch ships its own) the loader hands back that copy
// rather than mapping a second one.
#include "device_utils.cuh"
#include "kernels.hpp"

#include <atomic>
#include <cstdlib>
#include <string>

#include <cublas_v2.h>
#include <dlfcn.h>

#include <map>
#include <mutex>

namespace llaisys::kernels {

namespace {

struct CublasApi {
    cublasStatus_t (*create)(cublasHandle_t *) = nullptr;
    cublasStatus_t (*set_stream)(cublasHandle_t, cudaStream_t) = nullptr;
    cublasStatus_t (*gemm_ex)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void *, const void *,
                              cudaDataType, int, const void *, cudaDataType, int, const void *, void *, cudaDataType, int,
                              cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
    bool ok = false;
};

const CublasApi &cublas_api() {
    static CublasApi api = [] {
        CublasApi a;
        void *lib = nullptr;
        for (const char *name : {"libcublas.so.12", "libcublas.so", "/usr/local/cuda/lib64/libcublas.so.12"}) {
            lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (lib != nullptr) {
                break;
            }
        }
        if (lib == nullptr) {
            return a;
        }
        a.create = reinterpret_cast<decltype(a.create)>(dlsym(lib, "cublasCreate_v2"));
        a.set_stream = reinterpret_cast<decltype(a.set_stream)>(dlsym(lib, "cublasSetStream_v2"));
        a.gemm_ex = reinterpret_cast<decltype(a.gemm_ex)>(dlsym(lib, "cublasGemmEx"));
        a.ok = a.create != nullptr && a.set_stream != nullptr && a.gemm_ex != nullptr;
        return a;
    }();
    return api;
}

// One handle per (host thread, device): handles are not shared across threads and carry per-device state.
cublasHandle_t handle_for_current_device() {
    thread_local std::map<int, cublasHandle_t> handles;
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    auto it = handles.find(dev);
    if (it != handles.end()) {
        return it->second;
    }
    cublasHandle_t h = nullptr;
    const cublasStatus_t st = cublas_api().create(&h);
    ASSERT(st == CUBLAS_STATUS_SUCCESS, "cublasCreate failed with status " << int(st));
    handles.emplace(dev, h);
    return h;
}

std::atomic<int> g_linear_policy{0};

} // namespace

bool set_linear_policy(int policy) {
    if (policy < 0 || policy > 2) {
        return false;
    }
    g_linear_policy.store(policy, std::memory_order_relaxed);
    return true;
}

void linear(stream_t stream, llaisysDataType_t dtype, void *out, const void *in, const void *weight, const void *bias,
            size_t m, size_t n, size_t k, bool accumulate) {
    if (m == 0 || n == 0) {
        return;
    }
    // Decode-sized calls may take the hand-written streaming kernel (skinny_gemm_tc.cu). Measured on B200 against cuBLAS
    // (graph replays, weights rotated beyond L2): it wins where the activations are a small fraction of the traffic and K is
    // long enough to split over a cluster (8 x 8960 -> 1536: 12.5 vs 17.2 us); at 64 rows every CTA re-reads the
    // activations from L2 and cuBLAS's paired-CTA kernels are faster (64 x 1536 -> 17920: 16.5 vs 11.8 us), so those stay
    // with the library. set_linear_policy(1) takes the kernel wherever it applies, (2) never.
    const int policy = g_linear_policy.load(std::memory_order_relaxed);
    const bool force_tc = policy == 1, never_tc = policy == 2;
    const bool prefer_tc = m <= 16 && k >= 4096;
    if (!never_tc && (force_tc || prefer_tc) && m <= 128 &&
        linear_tc(stream, dtype, out, in, weight, m, n, k, accumulate, false)) {
        if (bias != nullptr) {
            bias_add(stream, dtype, out, bias, m, n);
        }
        return;
    }
    ASSERT(cublas_api().ok, "linear on NVIDIA needs cuBLAS (libcublas.so.12 was not found)");
    cudaDataType type;
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        type = CUDA_R_32F;
        break;
    case LLAISYS_DTYPE_F16:
        type = CUDA_R_16F;
        break;
    case LLAISYS_DTYPE_BF16:
        type = CUDA_R_16BF;
        break;
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
    cublasHandle_t h = handle_for_current_device();
    cublasStatus_t st = cublas_api().set_stream(h, static_cast<cudaStream_t>(stream));
    ASSERT(st == CUBLAS_STATUS_SUCCESS, "cublasSetStream failed with status " << int(st));
    // Row-major out[M, N] = in[M, K] . W[N, K]^T is column-major out^T[N, M] = W^T(as stored)[K, N]^T . in^T[K, M].
    const float alpha = 1.f, beta = accumulate ? 1.f : 0.f; // accumulate: out += in . W^T, one rounding of the sum
    st = cublas_api().gemm_ex(h, CUBLAS_OP_T, CUBLAS_OP_N, int(n), int(m), int(k), &alpha, weight, type, int(k), in, type,
                              int(k), &beta, out, type, int(n), CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    ASSERT(st == CUBLAS_STATUS_SUCCESS, "cublasGemmEx failed with status " << int(st));
    if (bias != nullptr) {
        bias_add(stream, dtype, out, bias, m, n);
    }
}

} // namespace llaisys::kernels
