// K3: log-sum-exp merge of partial attention results.
//
// parts is float [n_parts][n_rows][d + 2]: per row the locally normalised output o, then m (max scaled score)
// and l (sum of exp(score - m)). With M = max_p m_p and w_p = l_p exp(m_p - M),
//     out[r] = sum_p w_p o_p[r] / sum_p w_p.
// A part with l = 0 (it saw no keys; m = -inf) gets weight 0; if every part is empty the row is zero.
// One warp per row, lanes over d. HBM-bound: (n_parts * (d + 2) * 4 + d * elem) bytes per row.
#include "device_utils.cuh"
#include "kernels.hpp"

namespace llaisys::kernels {

namespace {

template <typename T>
__global__ void lse_merge_kernel(T *__restrict__ out, const float *__restrict__ parts, int n_parts, int n_rows,
                                 int d) {
    const int warps_per_block = blockDim.x >> 5;
    const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) {
        return;
    }
    const int64_t row_stride = d + 2;
    const int64_t part_stride = int64_t(n_rows) * row_stride;
    const float *base = parts + int64_t(row) * row_stride;
    float m_all = -INFINITY;
    for (int p = 0; p < n_parts; ++p) {
        const float l = base[p * part_stride + d + 1];
        if (l > 0.f) {
            m_all = fmaxf(m_all, base[p * part_stride + d]);
        }
    }
    float l_all = 0.f;
    for (int p = 0; p < n_parts; ++p) {
        const float l = base[p * part_stride + d + 1];
        if (l > 0.f) {
            l_all += l * expf(base[p * part_stride + d] - m_all);
        }
    }
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    for (int dim = lane; dim < d; dim += 32) {
        float o = 0.f;
        for (int p = 0; p < n_parts; ++p) {
            const float l = base[p * part_stride + d + 1];
            if (l > 0.f) {
                o = fmaf(l * expf(base[p * part_stride + d] - m_all), base[p * part_stride + dim], o);
            }
        }
        out[int64_t(row) * d + dim] = from_f32<T>(o * inv);
    }
}

} // namespace

void lse_merge(stream_t stream, llaisysDataType_t dtype, void *out, const float *parts, int32_t n_parts,
               int32_t n_rows, int32_t d) {
    if (n_rows <= 0 || d <= 0) {
        return;
    }
    auto s = static_cast<cudaStream_t>(stream);
    const int block = 128, grid = (n_rows + 3) / 4;
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        lse_merge_kernel<<<grid, block, 0, s>>>(static_cast<float *>(out), parts, n_parts, n_rows, d);
        break;
    case LLAISYS_DTYPE_F16:
        lse_merge_kernel<<<grid, block, 0, s>>>(static_cast<__half *>(out), parts, n_parts, n_rows, d);
        break;
    case LLAISYS_DTYPE_BF16:
        lse_merge_kernel<<<grid, block, 0, s>>>(static_cast<__nv_bfloat16 *>(out), parts, n_parts, n_rows, d);
        break;
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
    check_launch("lse_merge");
}

} // namespace llaisys::kernels
