// CUDA error checks. Two flavours: the legacy ABI throws (and so aborts the process, like every other
// misuse there); status-returning code uses LLAISYS_CUDA_TRY, which records the message and returns.
#pragma once

#include "../common/check.hpp"

#include <cuda_runtime.h>

#define LLAISYS_CUDA_CHECK(expr)                                                                         \
    do {                                                                                                 \
        cudaError_t err___ = (expr);                                                                     \
        if (err___ != cudaSuccess) {                                                                     \
            LLAISYS_RAISE_("CUDA error", cudaGetErrorName(err___) << ": " << cudaGetErrorString(err___)  \
                                                                  << " in " #expr,                       \
                           false);                                                                       \
        }                                                                                                \
    } while (0)
