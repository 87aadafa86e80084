/*
 * llaisys C ABI -- scalar types shared by every entry point.
 *
 * The numeric values below are the binary contract of the reference library
 * (reference: include/llaisys.h:23-28 device types, :31-52 data types,
 * :56 stream handle, :59-64 memcpy kinds) and are duplicated, by value, in its
 * Python frontend (reference: python/llaisys/libllaisys/llaisys_types.py:6-47).
 * A caller compiled against the reference headers can load this library unchanged.
 */
#ifndef LLAISYS_ABI_TYPES_H
#define LLAISYS_ABI_TYPES_H

#ifdef __cplusplus
#include <cstddef>
#include <cstdint>
#define LLAISYS_EXTERN_C extern "C"
#else
#include <stddef.h>
#include <stdint.h>
#define LLAISYS_EXTERN_C
#endif

#if defined(_WIN32)
#define LLAISYS_API __declspec(dllexport)
#else
#define LLAISYS_API __attribute__((visibility("default")))
#endif

/* Source compatibility with code written against the reference headers. */
#ifndef __export
#define __export LLAISYS_API
#endif
#ifndef __C
#define __C LLAISYS_EXTERN_C
#endif

/* Where a tensor lives. Values are consecutive; COUNT is one past the last. */
typedef enum {
    LLAISYS_DEVICE_CPU = 0,
    LLAISYS_DEVICE_NVIDIA = 1,
    LLAISYS_DEVICE_TYPE_COUNT
} llaisysDeviceType_t;

/* Element types. Only F32, F16 and BF16 carry arithmetic on the attention path;
 * I32/I64 appear as index tensors. */
typedef enum {
    LLAISYS_DTYPE_INVALID = 0,
    LLAISYS_DTYPE_BYTE = 1,
    LLAISYS_DTYPE_BOOL = 2,
    LLAISYS_DTYPE_I8 = 3,
    LLAISYS_DTYPE_I16 = 4,
    LLAISYS_DTYPE_I32 = 5,
    LLAISYS_DTYPE_I64 = 6,
    LLAISYS_DTYPE_U8 = 7,
    LLAISYS_DTYPE_U16 = 8,
    LLAISYS_DTYPE_U32 = 9,
    LLAISYS_DTYPE_U64 = 10,
    LLAISYS_DTYPE_F8 = 11,
    LLAISYS_DTYPE_F16 = 12,
    LLAISYS_DTYPE_F32 = 13,
    LLAISYS_DTYPE_F64 = 14,
    LLAISYS_DTYPE_C16 = 15,
    LLAISYS_DTYPE_C32 = 16,
    LLAISYS_DTYPE_C64 = 17,
    LLAISYS_DTYPE_C128 = 18,
    LLAISYS_DTYPE_BF16 = 19
} llaisysDataType_t;

/* Opaque stream handle: a cudaStream_t on NVIDIA, NULL on CPU. */
typedef void *llaisysStream_t;

typedef enum {
    LLAISYS_MEMCPY_H2H = 0,
    LLAISYS_MEMCPY_H2D = 1,
    LLAISYS_MEMCPY_D2H = 2,
    LLAISYS_MEMCPY_D2D = 3
} llaisysMemcpyKind_t;

#endif /* LLAISYS_ABI_TYPES_H */
