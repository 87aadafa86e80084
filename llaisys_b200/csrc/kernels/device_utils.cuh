// Small device helpers shared by the kernels: element conversion and launch checks.
#pragma once

#include "../device/cuda_check.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace llaisys::kernels {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

inline void check_launch(const char *what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        LLAISYS_RAISE_("CUDA launch failed", what << ": " << cudaGetErrorName(err) << ": " << cudaGetErrorString(err),
                       false);
    }
}

// Error-word bits written by kernels that skipped an access instead of faulting.
constexpr int kErrBadPage = 1;     // block-table entry outside [0, num_pages)
constexpr int kErrBadPosition = 2; // token position beyond the sequence's block table
constexpr int kErrBadSeq = 4;      // sequence row outside the table

} // namespace llaisys::kernels
