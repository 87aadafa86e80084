/*
 * llaisys C ABI -- tensor handles.
 *
 * Same 16 symbols, argument order and ownership rules as the reference
 * (reference: include/llaisys/tensor.h:9-65, thunks in src/llaisys/tensor.cc:5-96):
 *   - tensorCreate / tensorView / tensorPermute / tensorSlice return a NEW heap
 *     handle; the caller releases every handle with tensorDestroy. A handle keeps
 *     its storage alive, so a view may outlive the tensor it was taken from.
 *   - tensorGetShape / tensorGetStrides fill caller arrays of tensorGetNdim entries.
 *     Strides are in elements, not bytes.
 *   - Misuse prints "[ERROR] ..." to stderr and throws; the exception leaves the
 *     extern "C" frame and ends the process, exactly as the reference does
 *     (reference: src/utils/check.hpp:4-44).
 */
#ifndef LLAISYS_TENSOR_H
#define LLAISYS_TENSOR_H

#include "../llaisys.h"

typedef struct LlaisysTensor *llaisysTensor_t;

LLAISYS_EXTERN_C LLAISYS_API llaisysTensor_t tensorCreate(size_t *shape, size_t ndim, llaisysDataType_t dtype,
                                                          llaisysDeviceType_t device_type, int device_id);
LLAISYS_EXTERN_C LLAISYS_API void tensorDestroy(llaisysTensor_t tensor);

LLAISYS_EXTERN_C LLAISYS_API void *tensorGetData(llaisysTensor_t tensor);
LLAISYS_EXTERN_C LLAISYS_API size_t tensorGetNdim(llaisysTensor_t tensor);
LLAISYS_EXTERN_C LLAISYS_API void tensorGetShape(llaisysTensor_t tensor, size_t *shape);
LLAISYS_EXTERN_C LLAISYS_API void tensorGetStrides(llaisysTensor_t tensor, ptrdiff_t *strides);
LLAISYS_EXTERN_C LLAISYS_API llaisysDataType_t tensorGetDataType(llaisysTensor_t tensor);
LLAISYS_EXTERN_C LLAISYS_API llaisysDeviceType_t tensorGetDeviceType(llaisysTensor_t tensor);
LLAISYS_EXTERN_C LLAISYS_API int tensorGetDeviceId(llaisysTensor_t tensor);
LLAISYS_EXTERN_C LLAISYS_API void tensorDebug(llaisysTensor_t tensor);
LLAISYS_EXTERN_C LLAISYS_API uint8_t tensorIsContiguous(llaisysTensor_t tensor);

/* Copies numel*elem_size bytes from HOST memory at `data` into the tensor. */
LLAISYS_EXTERN_C LLAISYS_API void tensorLoad(llaisysTensor_t tensor, const void *data);

LLAISYS_EXTERN_C LLAISYS_API llaisysTensor_t tensorView(llaisysTensor_t tensor, size_t *shape, size_t ndim);
LLAISYS_EXTERN_C LLAISYS_API llaisysTensor_t tensorPermute(llaisysTensor_t tensor, size_t *order);
LLAISYS_EXTERN_C LLAISYS_API llaisysTensor_t tensorSlice(llaisysTensor_t tensor, size_t dim, size_t start, size_t end);

#endif /* LLAISYS_TENSOR_H */
