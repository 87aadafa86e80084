// add and rearrange on the device: both HBM-bound, one pass over the data.
#include "device_utils.cuh"
#include "kernels.hpp"

namespace llaisys::kernels {

namespace {

template <typename T>
__global__ void add_kernel(T *__restrict__ c, const T *__restrict__ a, const T *__restrict__ b, size_t n) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        c[i] = from_f32<T>(to_f32(a[i]) + to_f32(b[i]));
    }
}

constexpr int kMaxDims = 8;
struct RearrangeDims {
    unsigned long long shape[kMaxDims];
    long long dst_stride[kMaxDims];
    long long src_stride[kMaxDims];
    int ndim;
};

template <typename Word>
__global__ void rearrange_kernel(Word *__restrict__ dst, const Word *__restrict__ src, RearrangeDims dims,
                                 size_t total) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t rem = i;
        long long d_off = 0, s_off = 0;
        for (int k = dims.ndim - 1; k >= 0; --k) {
            const size_t idx = rem % dims.shape[k];
            rem /= dims.shape[k];
            d_off += (long long)idx * dims.dst_stride[k];
            s_off += (long long)idx * dims.src_stride[k];
        }
        dst[d_off] = src[s_off];
    }
}

int grid_for(size_t n, int block) {
    const size_t want = (n + block - 1) / block;
    const size_t cap = 148 * 16; // a few waves on 148 SMs; the loops are grid-strided
    return int(want < cap ? (want ? want : 1) : cap);
}

} // namespace

void fill_zero(stream_t stream, void *ptr, size_t bytes) {
    if (bytes == 0) {
        return;
    }
    LLAISYS_CUDA_CHECK(cudaMemsetAsync(ptr, 0, bytes, static_cast<cudaStream_t>(stream)));
}

void add(stream_t stream, llaisysDataType_t dtype, void *c, const void *a, const void *b, size_t n) {
    if (n == 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    const int block = 256, grid = grid_for(n, block);
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        add_kernel<<<grid, block, 0, s>>>(static_cast<float *>(c), static_cast<const float *>(a),
                                          static_cast<const float *>(b), n);
        break;
    case LLAISYS_DTYPE_F16:
        add_kernel<<<grid, block, 0, s>>>(static_cast<__half *>(c), static_cast<const __half *>(a),
                                          static_cast<const __half *>(b), n);
        break;
    case LLAISYS_DTYPE_BF16:
        add_kernel<<<grid, block, 0, s>>>(static_cast<__nv_bfloat16 *>(c), static_cast<const __nv_bfloat16 *>(a),
                                          static_cast<const __nv_bfloat16 *>(b), n);
        break;
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
    check_launch("add");
}

void rearrange(stream_t stream, size_t elem_size, size_t ndim, const size_t *shape, const ptrdiff_t *dst_strides,
               const ptrdiff_t *src_strides, void *dst, const void *src) {
    CHECK_ARGUMENT(ndim <= size_t(kMaxDims), "rearrange: at most 8 dimensions");
    RearrangeDims dims{};
    dims.ndim = int(ndim);
    size_t total = 1;
    for (size_t i = 0; i < ndim; ++i) {
        dims.shape[i] = shape[i];
        dims.dst_stride[i] = dst_strides[i];
        dims.src_stride[i] = src_strides[i];
        total *= shape[i];
    }
    if (total == 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    const int block = 256, grid = grid_for(total, block);
    switch (elem_size) {
    case 1:
        rearrange_kernel<<<grid, block, 0, s>>>(static_cast<uint8_t *>(dst), static_cast<const uint8_t *>(src), dims,
                                                total);
        break;
    case 2:
        rearrange_kernel<<<grid, block, 0, s>>>(static_cast<uint16_t *>(dst), static_cast<const uint16_t *>(src), dims,
                                                total);
        break;
    case 4:
        rearrange_kernel<<<grid, block, 0, s>>>(static_cast<uint32_t *>(dst), static_cast<const uint32_t *>(src), dims,
                                                total);
        break;
    case 8:
        rearrange_kernel<<<grid, block, 0, s>>>(static_cast<uint64_t *>(dst), static_cast<const uint64_t *>(src), dims,
                                                total);
        break;
    default:
        CHECK_ARGUMENT(false, "rearrange: element size must be 1, 2, 4 or 8 bytes");
    }
    check_launch("rearrange");
}

} // namespace llaisys::kernels
