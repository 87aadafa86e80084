// The operators around the attention path that a decode step of the model needs (specs: reference README.md:157-302):
// argmax, embedding, rms_norm, rope, swiglu and the bias add of linear. All HBM-bound, one pass over their data,
// f32 arithmetic with one rounding to the tensor dtype.
#include "device_utils.cuh"
#include "kernels.hpp"
#include "mma_utils.cuh"

#include <utility>

namespace llaisys::kernels {

namespace {

// A launch with programmatic stream serialisation, for kernels that wait for their predecessor (griddepcontrol.wait)
// before they touch anything: safe behind any kernel, and behind a long one it hides the launch.
template <typename... KArgs, typename... Args>
void launch_programmatic(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t s, Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    LLAISYS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...));
}

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

// ---- rms_norm: one CTA per row; 16-byte loads when the row allows, the row kept in registers between the passes --
template <typename T, int VEC, int PER_THREAD>
__global__ void rms_norm_vec_kernel(T *__restrict__ out, const T *__restrict__ in, const T *__restrict__ w, float eps, size_t d) {
    // launched programmatically: the grid may be scheduled under the tail of the kernel before it, touches nothing
    // until that kernel has completed, and only then lets its own successor be scheduled the same way (so whatever
    // starts early behind this grid can rely on everything before this grid's predecessor being complete)
    grid_dependency_wait();
    grid_launch_dependents();
    struct alignas(sizeof(T) * VEC) P {
        T v[VEC];
    };
    const size_t n_vec = d / VEC;
    const P *x = reinterpret_cast<const P *>(in + size_t(blockIdx.x) * d);
    P held[PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < PER_THREAD; ++r) {
        const size_t i = threadIdx.x + size_t(r) * blockDim.x;
        if (i < n_vec) {
            held[r] = x[i];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float v = to_f32(held[r].v[e]);
                ss = fmaf(v, v, ss);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    __shared__ float s_part[32];
    if ((threadIdx.x & 31) == 0) {
        s_part[threadIdx.x >> 5] = ss;
    }
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < int((blockDim.x + 31) >> 5); ++i) {
        tot += s_part[i]; // every thread sums the few partials in the same order
    }
    const float inv = rsqrtf(tot / float(d) + eps);
    P *y = reinterpret_cast<P *>(out + size_t(blockIdx.x) * d);
    const P *wv = reinterpret_cast<const P *>(w);
#pragma unroll
    for (int r = 0; r < PER_THREAD; ++r) {
        const size_t i = threadIdx.x + size_t(r) * blockDim.x;
        if (i < n_vec) {
            const P ww = wv[i];
            P o;
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                o.v[e] = from_f32<T>(to_f32(ww.v[e]) * to_f32(held[r].v[e]) * inv);
            }
            y[i] = o;
        }
    }
}

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

template <typename T, int VEC>
__global__ void swiglu_packed_kernel(T *__restrict__ out, const T *__restrict__ gu, size_t rows, size_t di) {
    grid_dependency_wait(); // (programmatic launch, as rms_norm_vec_kernel)
    grid_launch_dependents();
    struct alignas(sizeof(T) * VEC) P {
        T v[VEC];
    };
    const size_t per_row = di / VEC, total = rows * per_row;
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r = i / per_row, c = (i - r * per_row) * VEC;
        const P g = *reinterpret_cast<const P *>(gu + r * 2 * di + c);
        const P u = *reinterpret_cast<const P *>(gu + r * 2 * di + di + c);
        P o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float gv = to_f32(g.v[e]);
            o.v[e] = from_f32<T>(to_f32(u.v[e]) * (gv / (1.f + expf(-gv))));
        }
        *reinterpret_cast<P *>(out + r * di + c) = o;
    }
}

// ---- argmax over long rows: grid (splits, rows). A row's CTAs fold (value, index) into one 64-bit key with atomicMax
// (value in order-preserving bits above, inverted index below: the larger value wins, then the smaller index); the last
// CTA of the row to arrive writes the index and zeroes the row's key and counter for the next call.
__device__ __forceinline__ unsigned long long argmax_key(float v, size_t i) {
    const unsigned b = __float_as_uint(v);
    const unsigned ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return (static_cast<unsigned long long>(ord) << 32) | static_cast<unsigned long long>(0xffffffffu - unsigned(i));
}

template <typename T>
__global__ void argmax_split_kernel(int64_t *__restrict__ idx_out, const T *__restrict__ vals, size_t n,
                                    unsigned long long *__restrict__ keys, unsigned *__restrict__ counters) {
    const size_t row_i = blockIdx.y;
    const T *row = vals + row_i * n;
    const size_t chunk = (n + gridDim.x - 1) / gridDim.x;
    const size_t lo = size_t(blockIdx.x) * chunk, hi = lo + chunk < n ? lo + chunk : n;
    unsigned long long best = 0;
    for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = to_f32(row[i]);
        const unsigned long long key = v == v ? argmax_key(v, i) : 0ull; // NaN never wins
        best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    __shared__ unsigned long long s_best[32];
    if ((threadIdx.x & 31) == 0) {
        s_best[threadIdx.x >> 5] = best;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < int(blockDim.x >> 5); ++i) {
            best = s_best[i] > best ? s_best[i] : best;
        }
        atomicMax(keys + row_i, best);
        __threadfence();
        if (atomicAdd(counters + row_i, 1u) == gridDim.x - 1) {
            __threadfence();
            const unsigned long long win = atomicExch(keys + row_i, 0ull);
            counters[row_i] = 0u;
            idx_out[row_i] = win == 0ull ? 0 : int64_t(0xffffffffu - unsigned(win & 0xffffffffull));
        }
    }
}

int grid_for(size_t n, int block) {
    const size_t want = (n + block - 1) / block;
    const size_t cap = 148 * 16;
    return int(want < cap ? (want ? want : 1) : cap);
}

} // namespace

#define LLAISYS_CUDA_DISPATCH_FLOAT(dtype, ...)   \
    switch (dtype) {                              \
    case LLAISYS_DTYPE_F32: {                     \
        using T = float;                          \
        __VA_ARGS__;                              \
        break;                                    \
    }                                             \
    case LLAISYS_DTYPE_F16: {                     \
        using T = __half;                         \
        __VA_ARGS__;                              \
        break;                                    \
    }                                             \
    case LLAISYS_DTYPE_BF16: {                    \
        using T = __nv_bfloat16;                  \
        __VA_ARGS__;                              \
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
    auto aligned = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool ptrs_ok = aligned(out) && aligned(in) && aligned(weight);
    LLAISYS_CUDA_DISPATCH_FLOAT(dtype, {
        constexpr int kVec = 16 / int(sizeof(T));
        constexpr int kPerThread = 4;
        const size_t n_vec = d / kVec;
        if (ptrs_ok && d % kVec == 0 && n_vec <= size_t(1024) * kPerThread) {
            const size_t want = (n_vec + kPerThread - 1) / kPerThread;
            const unsigned block = unsigned(want <= 64 ? 64 : (want + 31) / 32 * 32);
            launch_programmatic(rms_norm_vec_kernel<T, kVec, kPerThread>, unsigned(rows), block, s, static_cast<T *>(out),
                                static_cast<const T *>(in), static_cast<const T *>(weight), eps, d);
        } else {
            rms_norm_kernel<T><<<unsigned(rows), 256, 0, s>>>(static_cast<T *>(out), static_cast<const T *>(in),
                                                               static_cast<const T *>(weight), eps, d);
        }
    });
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

void swiglu_packed(stream_t stream, llaisysDataType_t dtype, void *out, const void *gate_up, size_t rows, size_t di) {
    if (rows == 0 || di == 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    auto aligned = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool ptrs_ok = aligned(out) && aligned(gate_up);
    LLAISYS_CUDA_DISPATCH_FLOAT(dtype, {
        constexpr int kVec = 16 / int(sizeof(T));
        if (ptrs_ok && di % kVec == 0) {
            launch_programmatic(swiglu_packed_kernel<T, kVec>, unsigned(grid_for(rows * di / kVec, 256)), 256u, s,
                                static_cast<T *>(out), static_cast<const T *>(gate_up), rows, di);
        } else {
            launch_programmatic(swiglu_packed_kernel<T, 1>, unsigned(grid_for(rows * di, 256)), 256u, s, static_cast<T *>(out),
                                static_cast<const T *>(gate_up), rows, di);
        }
    });
    check_launch("swiglu_packed");
}

void argmax_rows_split(stream_t stream, llaisysDataType_t dtype, int64_t *idx_out, const void *vals, size_t rows, size_t n,
                       void *scratch) {
    if (rows == 0 || n == 0) {
        return;
    }
    CHECK_ARGUMENT(n < 0xffffffffull, "argmax: row too long for the packed key");
    auto s = static_cast<cudaStream_t>(stream);
    auto *keys = static_cast<unsigned long long *>(scratch);
    auto *counters = reinterpret_cast<unsigned *>(keys + rows);
    // enough CTAs to fill the GPU a few times over, at least 4096 elements each
    size_t splits = (n + 4095) / 4096;
    const size_t cap = (148 * 8 + rows - 1) / rows;
    splits = splits > cap ? cap : splits;
    splits = splits ? splits : 1;
    const dim3 grid{static_cast<unsigned>(splits), static_cast<unsigned>(rows), 1u};
    LLAISYS_CUDA_DISPATCH_FLOAT(dtype, (argmax_split_kernel<T><<<grid, 256, 0, s>>>(idx_out, static_cast<const T *>(vals), n,
                                                                                   keys, counters)));
    check_launch("argmax_split");
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
