// Element types: sizes, names, and software f16/bf16 <-> f32 conversion for host code.
//
// Host conversions follow the reference bit for bit where it defines them
// (src/utils/types.cpp:66-84: bf16 -> f32 is a 16-bit shift; f32 -> bf16 adds 0x7FFF plus the
// low kept bit, i.e. round to nearest even, with no NaN special case). Device code uses the CUDA
// intrinsics, which round the same way for every finite value.
#pragma once

#include "llaisys.h"

#include <cstdint>
#include <cstring>
#include <type_traits>

namespace llaisys {

struct fp16_t {
    uint16_t _v;
};
struct bf16_t {
    uint16_t _v;
};

namespace utils {

size_t dsize(llaisysDataType_t dtype);
const char *dtype_to_str(llaisysDataType_t dtype);

float _f16_to_f32(fp16_t h);
fp16_t _f32_to_f16(float f);

inline float _bf16_to_f32(bf16_t b) {
    uint32_t w = uint32_t(b._v) << 16;
    float f;
    std::memcpy(&f, &w, 4);
    return f;
}

inline bf16_t _f32_to_bf16(float f) {
    uint32_t w;
    std::memcpy(&w, &f, 4);
    w += 0x7FFFu + ((w >> 16) & 1u);
    return bf16_t{uint16_t(w >> 16)};
}

// cast<To>(from): any arithmetic type or fp16_t/bf16_t to any other, through float for the 16-bit types.
template <typename To, typename From>
inline To cast(From v) {
    if constexpr (std::is_same_v<To, From>) {
        return v;
    } else if constexpr (std::is_same_v<From, fp16_t>) {
        return cast<To>(_f16_to_f32(v));
    } else if constexpr (std::is_same_v<From, bf16_t>) {
        return cast<To>(_bf16_to_f32(v));
    } else if constexpr (std::is_same_v<To, fp16_t>) {
        return _f32_to_f16(static_cast<float>(v));
    } else if constexpr (std::is_same_v<To, bf16_t>) {
        return _f32_to_bf16(static_cast<float>(v));
    } else {
        return static_cast<To>(v);
    }
}

} // namespace utils
} // namespace llaisys
