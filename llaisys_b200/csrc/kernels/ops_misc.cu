// The operators around the attention path that a decode step of the model needs (specs: reference README.md:157-302):
// argmax, embedding, rms_norm, rope, swiglu and the bias add of linear. All HBM-bound, one pass over their data,
// f32 arithmetic with one rounding to the tensor dtype.
#include "device_utils.cuh"
#include "kernels.hpp"

namespace llaisys::kernels {

namespace {

// ---- argmax: one CTA per row, (value, index) pairs reduced with shuffles then through shared memory ----------------
template <typename T>
__global__ void argmax_rows_kernel(int64_t *__restrict__ idx_out, T *__restrict__ val_out, const T *__restrict__ vals,
                                   size_t n) {
    const T *row = vals + size_t(blockIdx.x) * n;
    float best = -INFINITY;
    size_t best_i = n; // n = "nothing yet"; smaller index wins among equal values
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = to_f32(row[i]);
        if (v > best || (v == best && i < best_i) || best_i == n) {
            best = v;
            best_i = i;
        }
    }
    auto better = [](float v, size_t i, float w, size_t j) { return v > w || (v == w && i < j); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, best, o);
        const unsigned long long j = __shfl_xor_sync(0xffffffffu, (unsigned long long)best_i, o);
        if (j != n && (best_i == n || better(w, j, best, best_i))) {
            best = w;
            best_i = j;
        }
    }
    __shared__ float s_v[32];
    __shared__ unsigned long long s_i[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        s_v[warp] = best;
        s_i[warp] = best_i;
    }
    __syncthreads();
    if (warp == 0) {
        const int n_warps = blockDim.x >> 5;
        best = lane < n_warps ? s_v[lane] : -INFINITY;
        best_i = lane < n_warps ? s_i[lane] : n;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float w = __shfl_xor_sync(0xffffffffu, best, o);
            const unsigned long long j = __shfl_xor_sync(0xffffffffu, (unsigned long long)best_i, o);
            if (j != n && (best_i == n || better(w, j, best, best_i))) {
                best = w;
                best_i = j;
            }
        }
        if (lane == 0) {
            idx_out[blockIdx.x] = int64_t(best_i == n ? 0 : best_i);
            if (val_out != nullptr) {
                val_out[blockIdx.x] = row[best_i == n ? 0 : best_i];
            }
        }
    }
}

// ---- embedding: 16-byte (or element-wise) row gather ---------------------------------------------------------------
__global__ void embedding_kernel(unsigned char *__restrict__ out, const int64_t *__restrict__ index,
                                 const unsigned char *__restrict__ weight, size_t row_bytes, size_t vocab) {
    const size_t i = blockIdx.x;
    long long src = index[i];
    if (src < 0 || size_t(src) >= vocab) {
        src = 0; // validated on the host where the indices are host-visible; never read out of range here
    }
    const unsigned char *s = weight + size_t(src) * row_bytes;
    unsigned char *d = out + i * row_bytes;
    if (row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(s) % 16 == 0) && (reinterpret_cast<uintptr_t>(d) % 16 == 0)) {
        for (size_t b = threadIdx.x * 16; b < row_bytes; b += size_t(blockDim.x) * 16) {
            *reinterpret_cast<uint4 *>(d + b) = *reinterpret_cast<const uint4 *>(s + b);
        }
    } else {
        for (size_t b = threadIdx.x; b < row_bytes; b += blockDim.x) {
            d[b] = s[b];
        }
    }
}

// ---- rms_norm: one CTA per row -------------------------------------------------------------------------------------
template <typename T>
__global__ void rms_norm_kernel(T *__restrict__ out, const T *__restrict__ in, const T *__restrict__ w, float eps, size_t d) {
    const T *x = in + size_t(blockIdx.x) * d;
    float ss = 0.f;
    for (size_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = to_f32(x[i]);
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    __shared__ float s_part[32];
    __shared__ float s_inv;
    if ((threadIdx.x & 31) == 0) {
        s_part[threadIdx.x >> 5] = ss;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < int(blockDim.x >> 5); ++i) {
            tot += s_part[i];
        }
        s_inv = rsqrtf(tot / float(d) + eps);
    }
    __syncthreads();
    const float inv = s_inv;
    for (size_t i = threadIdx.x; i < d; i += blockDim.x) {
        out[size_t(blockIdx.x) * d + i] = from_f32<T>(to_f32(w[i]) * to_f32(x[i]) * inv);
    }
}

// ---- rope ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kernel(T *__restrict__ out, const T *__restrict__ in, const int64_t *__restrict__ pos, float theta,
                            size_t heads, size_t d, size_t total_pairs) {
    const size_t half = d / 2;
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total_pairs; i += stride) {
        const size_t j = i % half;
        const size_t vec = i / half; // (token, head)
        const size_t s = vec / heads;
        const float ang = float(pos[s]) / powf(theta, 2.f * float(j) / float(d));
        float sn, cs;
        sincosf(ang, &sn, &cs);
        const float a = to_f32(in[vec * d + j]), b = to_f32(in[vec * d + j + half]);
        out[vec * d + j] = from_f32<T>(a * cs - b * sn);
        out[vec * d + j + half] = from_f32<T>(b * cs + a * sn);
    }
}

template <typename T>
__global__ void swiglu_kernel(T *__restrict__ out, const T *__restrict__ gate, const T *__restrict__ up, size_t n) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float g = to_f32(gate[i]);
        out[i] = from_f32<T>(to_f32(up[i]) * (g / (1.f + expf(-g))));
    }
}

template <typename T>
__global__ void bias_add_kernel(T *__restrict__ out, const T *__restrict__ bias, size_t n, size_t total) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        out[i] = from_f32<T>(to_f32(out[i]) + to_f32(bias[i % n]));
    }
}

int grid_for(size_t n, int block) {
    const size_t want = (n + block - 1) / block;
    const size_t cap = 148 * 16;
    return int(want < cap ? (want ? want : 1) : cap);
}

} // namespace

#define LLAISYS_CUDA_DISPATCH_FLOAT(dtype, CALL)  \
    switch (dtype) {                              \
    case LLAISYS_DTYPE_F32: {                     \
        using T = float;                          \
        CALL;                                     \
        break;                                    \
    }                                             \
    case LLAISYS_DTYPE_F16: {                     \
        using T = __half;                         \
        CALL;                                     \
        break;                                    \
    }                                             \
    case LLAISYS_DTYPE_BF16: {                    \
        using T = __nv_bfloat16;                  \
        CALL;                                     \
        break;                                    \
    }                                             \
    default:                                      \
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);    \
    }

void argmax_rows(stream_t stream, llaisysDataType_t dtype, int64_t *idx_out, void *val_out, const void *vals, size_t rows,
                 size_t n) {
    if (rows == 0 || n == 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    LLAISYS_CUDA_DISPATCH_FLOAT(dtype, (argmax_rows_kernel<T><<<unsigned(rows), 1024, 0, s>>>(
                                           idx_out, static_cast<T *>(val_out), static_cast<const T *>(vals), n)));
    check_launch("argmax");
}

void embedding(stream_t stream, size_t elem_size, void *out, const int64_t *index, const void *weight, size_t n, size_t d,
               size_t vocab) {
    if (n == 0 || d == 0) {
        return;
    }
    embedding_kernel<<<unsigned(n), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<unsigned char *>(out), index, static_cast<const unsigned char *>(weight), d * elem_size, vocab);
    check_launch("embedding");
}

void rms_norm(stream_t stream, llaisysDataType_t dtype, void *out, const void *in, const void *weight, float eps, size_t rows,
              size_t d) {
    if (rows == 0 || d == 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    LLAISYS_CUDA_DISPATCH_FLOAT(dtype, (rms_norm_kernel<T><<<unsigned(rows), 256, 0, s>>>(
                                           static_cast<T *>(out), static_cast<const T *>(in), static_cast<const T *>(weight), eps, d)));
    check_launch("rms_norm");
}

void rope(stream_t stream, llaisysDataType_t dtype, void *out, const void *in, const int64_t *pos, float theta, size_t seq,
          size_t heads, size_t d) {
    const size_t pairs = seq * heads * (d / 2);
    if (pairs == 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    LLAISYS_CUDA_DISPATCH_FLOAT(dtype, (rope_kernel<T><<<grid_for(pairs, 256), 256, 0, s>>>(
                                           static_cast<T *>(out), static_cast<const T *>(in), pos, theta, heads, d, pairs)));
    check_launch("rope");
}

void swiglu(stream_t stream, llaisysDataType_t dtype, void *out, const void *gate, const void *up, size_t n) {
    if (n == 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    LLAISYS_CUDA_DISPATCH_FLOAT(dtype, (swiglu_kernel<T><<<grid_for(n, 256), 256, 0, s>>>(
                                           static_cast<T *>(out), static_cast<const T *>(gate), static_cast<const T *>(up), n)));
    check_launch("swiglu");
}

void bias_add(stream_t stream, llaisysDataType_t dtype, void *out, const void *bias, size_t rows, size_t n) {
    if (rows == 0 || n == 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    LLAISYS_CUDA_DISPATCH_FLOAT(dtype, (bias_add_kernel<T><<<grid_for(rows * n, 256), 256, 0, s>>>(
                                           static_cast<T *>(out), static_cast<const T *>(bias), n, rows * n)));
    check_launch("bias_add");
}

} // namespace llaisys::kernels
