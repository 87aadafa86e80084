#include "check.hpp"
#include "dtypes.hpp"

#include <iostream>

namespace llaisys::detail {

void raise(const char *kind, const std::string &what, const char *func, const char *file, int line,
           bool invalid_argument) {
    std::string text = kind;
    if (!what.empty()) {
        text += ": ";
        text += what;
    }
    std::cerr << "[ERROR] " << text << " from " << func << " at " << file << ":" << line << "." << std::endl;
    if (invalid_argument) {
        throw std::invalid_argument(text);
    }
    throw std::runtime_error(text);
}

} // namespace llaisys::detail

namespace llaisys::utils {

namespace {
struct DtypeInfo {
    llaisysDataType_t dtype;
    size_t size;
    const char *name;
};
// Sizes and names as the reference reports them (src/utils/types.hpp:18-108).
constexpr DtypeInfo kDtypes[] = {
    {LLAISYS_DTYPE_BYTE, 1, "byte"},       {LLAISYS_DTYPE_BOOL, 1, "bool"},       {LLAISYS_DTYPE_I8, 1, "int8"},
    {LLAISYS_DTYPE_I16, 2, "int16"},       {LLAISYS_DTYPE_I32, 4, "int32"},       {LLAISYS_DTYPE_I64, 8, "int64"},
    {LLAISYS_DTYPE_U8, 1, "uint8"},        {LLAISYS_DTYPE_U16, 2, "uint16"},      {LLAISYS_DTYPE_U32, 4, "uint32"},
    {LLAISYS_DTYPE_U64, 8, "uint64"},      {LLAISYS_DTYPE_F8, 1, "float8"},       {LLAISYS_DTYPE_F16, 2, "float16"},
    {LLAISYS_DTYPE_F32, 4, "float32"},     {LLAISYS_DTYPE_F64, 8, "float64"},     {LLAISYS_DTYPE_C16, 2, "complex16"},
    {LLAISYS_DTYPE_C32, 4, "complex32"},   {LLAISYS_DTYPE_C64, 8, "complex64"},   {LLAISYS_DTYPE_C128, 16, "complex128"},
    {LLAISYS_DTYPE_BF16, 2, "bfloat16"},
};

const DtypeInfo &lookup(llaisysDataType_t dtype) {
    for (const auto &e : kDtypes) {
        if (e.dtype == dtype) {
            return e;
        }
    }
    throw std::invalid_argument("Unsupported or invalid data type.");
}
} // namespace

size_t dsize(llaisysDataType_t dtype) { return lookup(dtype).size; }
const char *dtype_to_str(llaisysDataType_t dtype) { return lookup(dtype).name; }

// IEEE binary16 -> binary32: exact for every input, subnormals included.
float _f16_to_f32(fp16_t h) {
    const uint32_t sign = uint32_t(h._v & 0x8000u) << 16;
    uint32_t exp = (h._v >> 10) & 0x1Fu;
    uint32_t man = h._v & 0x3FFu;
    uint32_t w;
    if (exp == 0x1Fu) {
        w = sign | 0x7F800000u | (man << 13); // inf / nan, payload kept
    } else if (exp != 0) {
        w = sign | ((exp + 112u) << 23) | (man << 13);
    } else if (man == 0) {
        w = sign;
    } else {
        // subnormal: shift the leading one up to bit 10 and rebias
        int e = 113;
        while ((man & 0x400u) == 0) {
            man <<= 1;
            --e;
        }
        w = sign | (uint32_t(e) << 23) | ((man & 0x3FFu) << 13);
    }
    float f;
    std::memcpy(&f, &w, 4);
    return f;
}

// binary32 -> binary16, round to nearest even (what the CUDA conversion intrinsics and torch do).
// The reference's host helper truncates the mantissa instead (src/utils/types.cpp:35-64); rounding
// keeps the CPU and GPU backends of this library bit-identical on conversion and halves the error.
fp16_t _f32_to_f16(float f) {
    uint32_t w;
    std::memcpy(&w, &f, 4);
    const uint16_t sign = uint16_t((w >> 16) & 0x8000u);
    const uint32_t abs = w & 0x7FFFFFFFu;
    if (abs >= 0x7F800000u) { // inf / nan
        return fp16_t{uint16_t(sign | (abs > 0x7F800000u ? 0x7E00u : 0x7C00u))};
    }
    if (abs >= 0x477FF000u) { // >= 65520 rounds to infinity
        return fp16_t{uint16_t(sign | 0x7C00u)};
    }
    if (abs < 0x33000001u) { // <= 2^-25 rounds to zero
        return fp16_t{sign};
    }
    const int32_t e = int32_t(abs >> 23) - 127;
    uint32_t man = (abs & 0x7FFFFFu) | 0x800000u; // 24-bit significand
    // number of low bits dropped: 13 for normals, more for subnormal results
    const int shift = (e >= -14) ? 13 : (13 + (-14 - e));
    const uint32_t kept = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    uint32_t r = kept + ((rem > half || (rem == half && (kept & 1u))) ? 1u : 0u);
    uint32_t bits;
    if (e >= -14) {
        // kept has the implicit one at bit 10; adding the biased exponent minus one absorbs it, and a
        // carry out of the mantissa bumps the exponent by itself.
        bits = (uint32_t(e + 15 - 1) << 10) + r;
    } else {
        bits = r; // subnormal (a carry to 0x400 is the smallest normal, also correct)
    }
    return fp16_t{uint16_t(sign | bits)};
}

} // namespace llaisys::utils
