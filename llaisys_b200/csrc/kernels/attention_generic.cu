// Generic attention over a paged or contiguous K/V view: any of F32 / F16 / BF16, head_dim <= 256, any GQA
// ratio, any page size, decode or ragged causal chunks.
//
// One CTA of four warps per (query row, query head). Keys are dealt to warps in blocks of 32; inside a warp
// each lane scores one key (a full dot product against the query held in shared memory), the warp folds the 32
// scores into its running (max, sum) with shuffles, and the P.V update walks the 32 keys with every lane
// owning head_dim / 32 output dimensions, so V rows are read coalesced. The four warps are merged through
// shared memory at the end. All arithmetic is f32 with exact expf: this kernel is the on-device statement of
// the operator's definition (reference: test/ops/self_attention.py:11-28) that the specialised kernels are
// checked against, and the kernel behind the legacy operator for shapes those do not cover.
#include "device_utils.cuh"
#include "kernels.hpp"

#include <cfloat>

namespace llaisys::kernels {

namespace {

constexpr int kWarps = 4;
constexpr int kMaxDimsPerLane = 8; // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
    attention_generic_kernel(KVView kv, AttnBatch batch, const T *__restrict__ q, float scale, T *__restrict__ out,
                             float *__restrict__ part, int32_t *error_flag) {
    extern __shared__ float smem[];
    const int d = kv.d;
    float *q_s = smem;                    // [d] query, pre-multiplied by scale
    float *acc_s = smem + d;              // [kWarps][d]
    float *m_s = acc_s + kWarps * d;      // [kWarps]
    float *l_s = m_s + kWarps;            // [kWarps]

    const int row = blockIdx.x;
    const int h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which sequence does this query row belong to, and how many keys may it see
    int seq, t, q_len;
    if (batch.q_starts != nullptr) {
        int lo = 0, hi = batch.n_seqs - 1;
        while (lo < hi) { // last seq with q_starts[seq] <= row
            const int mid = (lo + hi + 1) >> 1;
            if (batch.q_starts[mid] <= row) {
                lo = mid;
            } else {
                hi = mid - 1;
            }
        }
        seq = lo;
        t = row - batch.q_starts[seq];
        q_len = batch.q_starts[seq + 1] - batch.q_starts[seq];
    } else {
        seq = row / batch.const_q_len;
        t = row - seq * batch.const_q_len;
        q_len = batch.const_q_len;
    }
    const int kv_len = batch.kv_lens ? batch.kv_lens[seq] : batch.const_kv_len;
    int visible = kv_len - q_len + t + 1; // causal offset: query t sees keys j <= t + (kv_len - q_len)
    visible = visible < 0 ? 0 : (visible > kv_len ? kv_len : visible);
    const int seq_row = batch.seq_ids ? batch.seq_ids[seq] : seq;
    const int kvh = h / (batch.nh / kv.nkvh);

    const T *q_row = q + (int64_t(row) * batch.nh + h) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        q_s[i] = to_f32(q_row[i]) * scale;
    }
    __syncthreads();

    const T *k_base = static_cast<const T *>(kv.k_base) + int64_t(kvh) * kv.head_stride;
    const T *v_base = static_cast<const T *>(kv.v_base) + int64_t(kvh) * kv.head_stride;

    float m = -INFINITY, l = 0.f;
    float acc[kMaxDimsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
        acc[i] = 0.f;
    }

    for (int base = warp * 32; base < visible; base += kWarps * 32) {
        const int j = base + lane;
        bool valid = j < visible;
        int64_t row_off = 0;
        if (valid) {
            const int blk = j / kv.page_size;
            int page = blk;
            if (kv.block_table != nullptr) {
                page = kv.block_table[int64_t(seq_row) * kv.table_stride + blk];
            }
            if (page < 0 || page >= kv.num_pages) {
                atomicOr(error_flag, kErrBadPage);
                valid = false;
            } else {
                row_off = int64_t(page) * kv.page_stride + int64_t(j - blk * kv.page_size) * kv.token_stride;
            }
        }
        float s = -INFINITY;
        if (valid) {
            const T *k_row = k_base + row_off;
            float dot = 0.f;
            for (int i = 0; i < d; ++i) {
                dot = fmaf(q_s[i], to_f32(k_row[i]), dot);
            }
            s = dot;
        }
        float mx = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (mx == -INFINITY) {
            continue; // no usable key in this block (warp-uniform)
        }
        const float m_new = fmaxf(m, mx);
        const float alpha = expf(m - m_new); // m = -inf on the first block gives 0
        const float p = valid ? expf(s - m_new) : 0.f;
        float p_sum = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            p_sum += __shfl_xor_sync(0xffffffffu, p_sum, o);
        }
        l = l * alpha + p_sum;
        m = m_new;
#pragma unroll
        for (int i = 0; i < kMaxDimsPerLane; ++i) {
            acc[i] *= alpha;
        }
        const int n_here = min(32, visible - base);
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int64_t off = __shfl_sync(0xffffffffu, row_off, jj);
            if (pj == 0.f) {
                continue; // skipped page or underflow (warp-uniform)
            }
            const T *v_row = v_base + off;
#pragma unroll
            for (int i = 0; i < kMaxDimsPerLane; ++i) {
                const int dim = lane + 32 * i;
                if (dim < d) {
                    acc[i] = fmaf(pj, to_f32(v_row[dim]), acc[i]);
                }
            }
        }
    }

    // merge the four warps
    if (lane == 0) {
        m_s[warp] = m;
        l_s[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int dim = lane + 32 * i;
        if (dim < d) {
            acc_s[warp * d + dim] = acc[i];
        }
    }
    __syncthreads();
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        m_all = fmaxf(m_all, m_s[w]);
    }
    float l_all = 0.f;
    float w_scale[kWarps];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        w_scale[w] = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - m_all);
        l_all += l_s[w] * w_scale[w];
    }
    const float inv_l = l_all > 0.f ? 1.f / l_all : 0.f;
    const int64_t o_row = int64_t(row) * batch.nh + h;
    for (int dim = threadIdx.x; dim < d; dim += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            o += acc_s[w * d + dim] * w_scale[w];
        }
        o *= inv_l;
        if (part != nullptr) {
            part[o_row * (d + 2) + dim] = o;
        } else {
            out[o_row * d + dim] = from_f32<T>(o);
        }
    }
    if (part != nullptr && threadIdx.x == 0) {
        part[o_row * (d + 2) + d] = m_all;
        part[o_row * (d + 2) + d + 1] = l_all;
    }
}

template <typename T>
void launch(cudaStream_t s, const KVView &kv, const AttnBatch &batch, const void *q, float scale, const AttnOut &out,
            int32_t *error_flag) {
    const dim3 grid(unsigned(batch.total_q), unsigned(batch.nh));
    const size_t smem = (size_t(kv.d) * (1 + kWarps) + 2 * kWarps) * sizeof(float);
    attention_generic_kernel<T><<<grid, kWarps * 32, smem, s>>>(kv, batch, static_cast<const T *>(q), scale,
                                                                static_cast<T *>(out.out), out.part, error_flag);
}

} // namespace

void attention_generic(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                       const void *q, float scale, const AttnOut &out, int32_t *error_flag) {
    if (batch.total_q <= 0 || batch.nh <= 0) {
        return;
    }
    CHECK_ARGUMENT(kv.d > 0 && kv.d <= 32 * kMaxDimsPerLane, "attention: head_dim must be in [1, 256]");
    CHECK_ARGUMENT(kv.nkvh > 0 && batch.nh % kv.nkvh == 0, "attention: nh must be a multiple of nkvh");
    CHECK_ARGUMENT(batch.nh <= 65535, "attention: too many heads for one launch");
    auto s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        launch<float>(s, kv, batch, q, scale, out, error_flag);
        break;
    case LLAISYS_DTYPE_F16:
        launch<__half>(s, kv, batch, q, scale, out, error_flag);
        break;
    case LLAISYS_DTYPE_BF16:
        launch<__nv_bfloat16>(s, kv, batch, q, scale, out, error_flag);
        break;
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
    check_launch("attention_generic");
}

} // namespace llaisys::kernels
