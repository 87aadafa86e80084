// Operator layer: argument checks, then dispatch on the device type of the output tensor -- the pattern of the
// reference's one worked operator (src/ops/add/op.cpp:9-34): CPU tensors run the CPU backend directly; anything
// else makes its device current and launches on that runtime's stream. A device tensor never runs on the host.
#include "ops.hpp"

#include "../common/check.hpp"
#include "../common/dtypes.hpp"
#include "../cpu/cpu_kernels.hpp"
#ifdef ENABLE_NVIDIA_API
#include "../kernels/kernels.hpp"
#include "../kv/paged_kv.hpp"
#include "llaisys/paged_kv.h"

#include <map>
#endif

namespace llaisys::ops {

namespace {
// Makes the tensor's device current and returns the stream operators queue on.
llaisysStream_t enter_device(const Tensor &t) {
    auto &ctx = core::context();
    ctx.setDevice(t.deviceType(), t.deviceId());
    return ctx.runtime().stream();
}

#ifdef ENABLE_NVIDIA_API
// The legacy operator has no cache object to own split-KV scratch, so each host thread keeps one set per
// device, grown on demand. Blocks come from the runtime's cache and are used on its stream only.
struct OperatorScratch {
    core::storage_t partials, counters, error;
    size_t partials_floats = 0, counters_len = 0;
};

void nvidia_self_attention(llaisysStream_t stream, llaisysDataType_t dtype, const kernels::KVView &view,
                           const kernels::AttnBatch &batch, const void *q, float scale, const kernels::AttnOut &out) {
    thread_local std::map<int, OperatorScratch> per_device;
    auto &rt = core::context().runtime();
    OperatorScratch &sc = per_device[rt.deviceId()];
    if (!sc.error) {
        sc.error = rt.allocateDeviceStorage(sizeof(int32_t));
        kernels::fill_zero(stream, sc.error->memory(), sizeof(int32_t));
    }
    kernels::AttnScratch scratch;
    scratch.error_flag = reinterpret_cast<int32_t *>(sc.error->memory());
    const bool chunk = batch.const_q_len >= 16 && view.d == 128 &&
                       (dtype == LLAISYS_DTYPE_BF16 || dtype == LLAISYS_DTYPE_F16); // tensor-core kernel: split tiles
    if (batch.const_q_len == 1 || chunk) {
        size_t floats = 0, counters = 0;
        if (chunk) {
            kernels::attention_prefill_tc_scratch(&floats, &counters);
        } else {
            kernels::attention_decode_split_scratch(batch.n_seqs, batch.nh, view.nkvh, view.d, batch.max_kv_len, &floats,
                                                    &counters);
        }
        if (floats > sc.partials_floats) {
            sc.partials = rt.allocateDeviceStorage(floats * sizeof(float));
            sc.partials_floats = floats;
        }
        if (counters > sc.counters_len) {
            sc.counters = rt.allocateDeviceStorage(counters * sizeof(int32_t));
            sc.counters_len = counters;
            kernels::fill_zero(stream, sc.counters->memory(), sc.counters->size());
        }
        scratch.partials = sc.partials ? reinterpret_cast<float *>(sc.partials->memory()) : nullptr;
        scratch.partials_floats = sc.partials_floats;
        scratch.counters = sc.counters ? reinterpret_cast<int32_t *>(sc.counters->memory()) : nullptr;
        scratch.counters_len = sc.counters_len;
    }
    kv::run_attention_nvidia(stream, dtype, view, batch, q, scale, out, scratch);
}
#endif

} // namespace

void add(tensor_t c, tensor_t a, tensor_t b) {
    CHECK_SAME_DEVICE(c, a, b);
    CHECK_SAME_SHAPE(c->shape(), a->shape(), b->shape());
    CHECK_SAME_DTYPE(c->dtype(), a->dtype(), b->dtype());
    ASSERT(c->isContiguous() && a->isContiguous() && b->isContiguous(), "Add: all tensors must be contiguous.");

    switch (c->deviceType()) {
    case LLAISYS_DEVICE_CPU:
        return cpu::add(c->dtype(), c->data(), a->data(), b->data(), c->numel());
#ifdef ENABLE_NVIDIA_API
    case LLAISYS_DEVICE_NVIDIA:
        return kernels::add(enter_device(*c), c->dtype(), c->data(), a->data(), b->data(), c->numel());
#endif
    default:
        EXCEPTION_UNSUPPORTED_DEVICE;
    }
}

void rearrange_raw(Tensor &dst, const Tensor &src) {
    CHECK_ARGUMENT(dst.deviceType() == src.deviceType() && dst.deviceId() == src.deviceId(),
                   "rearrange: tensors must be on the same device");
    CHECK_SAME_SHAPE(dst.shape(), src.shape());
    CHECK_SAME_DTYPE(dst.dtype(), src.dtype());
    switch (dst.deviceType()) {
    case LLAISYS_DEVICE_CPU:
        return cpu::rearrange(dst.elementSize(), dst.ndim(), dst.shape().data(), dst.strides().data(),
                              src.strides().data(), dst.data(), src.data());
#ifdef ENABLE_NVIDIA_API
    case LLAISYS_DEVICE_NVIDIA:
        return kernels::rearrange(enter_device(dst), dst.elementSize(), dst.ndim(), dst.shape().data(),
                                  dst.strides().data(), src.strides().data(), dst.data(), src.data());
#endif
    default:
        EXCEPTION_UNSUPPORTED_DEVICE;
    }
}

void rearrange(tensor_t out, tensor_t in) { rearrange_raw(*out, *in); }

// attn_val [qlen, nh, dv], q [qlen, nh, d], k [total, nkvh, d], v [total, nkvh, dv]; d == dv here (the pool and
// the kernels keep one head_dim). Causal with the cache offset: query i sees keys j <= i + (total - qlen)
// (reference: test/ops/self_attention.py:18, README.md:244-266).
void self_attention(tensor_t attn_val, tensor_t q, tensor_t k, tensor_t v, float scale) {
    CHECK_SAME_DEVICE(attn_val, q, k, v);
    CHECK_SAME_DTYPE(attn_val->dtype(), q->dtype(), k->dtype(), v->dtype());
    CHECK_ARGUMENT(attn_val->ndim() == 3 && q->ndim() == 3 && k->ndim() == 3 && v->ndim() == 3,
                   "SelfAttention: all tensors must be 3-dimensional");
    ASSERT(attn_val->isContiguous() && q->isContiguous() && k->isContiguous() && v->isContiguous(),
           "SelfAttention: all tensors must be contiguous.");
    const size_t qlen = q->shape()[0], nh = q->shape()[1], d = q->shape()[2];
    const size_t total = k->shape()[0], nkvh = k->shape()[1];
    CHECK_ARGUMENT(k->shape()[2] == d, "SelfAttention: q and k head dims differ");
    CHECK_SAME_SHAPE(k->shape(), v->shape()); // dv == d
    CHECK_SAME_SHAPE(attn_val->shape(), q->shape());
    CHECK_ARGUMENT(nkvh > 0 && nh % nkvh == 0, "SelfAttention: nhead must be a multiple of nkvhead");
    CHECK_ARGUMENT(total >= qlen, "SelfAttention: total_len must cover the queries");
    if (qlen == 0) {
        return;
    }

    // The contiguous K/V tensors seen as a one-sequence cache: block b is page b, rows interleave the heads.
    kernels::KVView view;
    view.k_base = k->data();
    view.v_base = v->data();
    view.page_size = 16;
    view.page_stride = int64_t(view.page_size) * int64_t(nkvh * d);
    view.head_stride = int64_t(d);
    view.token_stride = int64_t(nkvh * d);
    view.block_table = nullptr;
    view.num_pages = int32_t((total + view.page_size - 1) / view.page_size);
    view.nkvh = int32_t(nkvh);
    view.d = int32_t(d);

    kernels::AttnBatch batch;
    batch.n_seqs = 1;
    batch.const_kv_len = int32_t(total);
    batch.const_q_len = int32_t(qlen);
    batch.total_q = int32_t(qlen);
    batch.max_q_len = int32_t(qlen);
    batch.max_kv_len = int32_t(total);
    batch.nh = int32_t(nh);

    kernels::AttnOut out;
    out.out = attn_val->data();

    switch (attn_val->deviceType()) {
    case LLAISYS_DEVICE_CPU:
        cpu::attention(q->dtype(), view, batch, q->data(), scale, out);
        kv::noteAttentionKernel(LLAISYS_KERNEL_CPU);
        return;
#ifdef ENABLE_NVIDIA_API
    case LLAISYS_DEVICE_NVIDIA: {
        llaisysStream_t stream = enter_device(*attn_val);
        return nvidia_self_attention(stream, q->dtype(), view, batch, q->data(), scale, out);
    }
#endif
    default:
        EXCEPTION_UNSUPPORTED_DEVICE;
    }
}

// ---- the remaining operators of the ABI (stubs in the reference: src/ops/*/op.cpp:4-6; specs README.md:157-302) ----

#ifdef ENABLE_NVIDIA_API
#define LLAISYS_ON_DEVICE(TENSOR, CPU_CALL, CUDA_CALL)             \
    switch ((TENSOR)->deviceType()) {                              \
    case LLAISYS_DEVICE_CPU:                                       \
        CPU_CALL;                                                  \
        return;                                                    \
    case LLAISYS_DEVICE_NVIDIA: {                                  \
        llaisysStream_t stream = enter_device(*(TENSOR));          \
        CUDA_CALL;                                                 \
        return;                                                    \
    }                                                              \
    default:                                                       \
        EXCEPTION_UNSUPPORTED_DEVICE;                              \
    }
#else
#define LLAISYS_ON_DEVICE(TENSOR, CPU_CALL, CUDA_CALL) \
    switch ((TENSOR)->deviceType()) {                  \
    case LLAISYS_DEVICE_CPU:                           \
        CPU_CALL;                                      \
        return;                                        \
    default:                                           \
        EXCEPTION_UNSUPPORTED_DEVICE;                  \
    }
#endif

// vals 1-D [n] -> max_idx [1] int64, max_val [1] of the dtype of vals (reference: README.md:157-167)
void argmax(tensor_t max_idx, tensor_t max_val, tensor_t vals) {
    CHECK_SAME_DEVICE(max_idx, max_val, vals);
    CHECK_ARGUMENT(max_idx->dtype() == LLAISYS_DTYPE_I64, "Argmax: max_idx must be int64");
    CHECK_SAME_DTYPE(max_val->dtype(), vals->dtype());
    CHECK_ARGUMENT(max_idx->numel() == 1 && max_val->numel() == 1 && vals->numel() >= 1, "Argmax: shapes");
    ASSERT(vals->isContiguous(), "Argmax: vals must be contiguous.");
    LLAISYS_ON_DEVICE(vals,
                      cpu::argmax_rows(vals->dtype(), reinterpret_cast<int64_t *>(max_idx->data()), max_val->data(),
                                       vals->data(), 1, vals->numel()),
                      kernels::argmax_rows(stream, vals->dtype(), reinterpret_cast<int64_t *>(max_idx->data()),
                                           max_val->data(), vals->data(), 1, vals->numel()));
}

// out [n, d] = weight[index[n], :] (reference: README.md:169-177)
void embedding(tensor_t out, tensor_t index, tensor_t weight) {
    CHECK_SAME_DEVICE(out, index, weight);
    CHECK_ARGUMENT(index->dtype() == LLAISYS_DTYPE_I64, "Embedding: index must be int64");
    CHECK_SAME_DTYPE(out->dtype(), weight->dtype());
    CHECK_ARGUMENT(index->ndim() == 1 && out->ndim() == 2 && weight->ndim() == 2, "Embedding: index 1-D, out and weight 2-D");
    CHECK_ARGUMENT(out->shape()[0] == index->shape()[0] && out->shape()[1] == weight->shape()[1], "Embedding: shapes");
    ASSERT(out->isContiguous() && index->isContiguous() && weight->isContiguous(), "Embedding: tensors must be contiguous.");
    const size_t n = index->shape()[0], d = weight->shape()[1], vocab = weight->shape()[0];
    LLAISYS_ON_DEVICE(out,
                      cpu::embedding(out->elementSize(), out->data(), reinterpret_cast<const int64_t *>(index->data()),
                                     weight->data(), n, d, vocab),
                      kernels::embedding(stream, out->elementSize(), out->data(),
                                         reinterpret_cast<const int64_t *>(index->data()), weight->data(), n, d, vocab));
}

// out [M, N] = in [M, K] . weight [N, K]^T + bias [N]; bias may be null (reference: README.md:179-196)
void linear(tensor_t out, tensor_t in, tensor_t weight, tensor_t bias) { linear_ex(out, in, weight, bias, false); }

// accumulate: out += in . weight^T (+ bias), the sum rounded once -- a decoder block's residual add folded into its
// projection. No counterpart in the reference.
void linear_ex(tensor_t out, tensor_t in, tensor_t weight, tensor_t bias, bool accumulate) {
    CHECK_SAME_DEVICE(out, in, weight);
    CHECK_SAME_DTYPE(out->dtype(), in->dtype(), weight->dtype());
    CHECK_ARGUMENT(out->ndim() == 2 && in->ndim() == 2 && weight->ndim() == 2, "Linear: tensors must be 2-D");
    const size_t m = in->shape()[0], k = in->shape()[1], n = weight->shape()[0];
    CHECK_ARGUMENT(weight->shape()[1] == k && out->shape()[0] == m && out->shape()[1] == n, "Linear: shapes");
    ASSERT(out->isContiguous() && in->isContiguous() && weight->isContiguous(), "Linear: tensors must be contiguous.");
    const std::byte *bias_ptr = nullptr;
    if (bias) {
        CHECK_SAME_DEVICE(out, bias);
        CHECK_SAME_DTYPE(out->dtype(), bias->dtype());
        CHECK_ARGUMENT(bias->numel() == n, "Linear: bias must have one element per output column");
        ASSERT(bias->isContiguous(), "Linear: bias must be contiguous.");
        bias_ptr = bias->data();
    }
    LLAISYS_ON_DEVICE(out, cpu::linear(out->dtype(), out->data(), in->data(), weight->data(), bias_ptr, m, n, k, accumulate),
                      kernels::linear(stream, out->dtype(), out->data(), in->data(), weight->data(), bias_ptr, m, n, k, accumulate));
}

// per row: out = weight * in / sqrt(mean(in^2) + eps) (reference: README.md:198-213)
void rms_norm(tensor_t out, tensor_t in, tensor_t weight, float eps) {
    CHECK_SAME_DEVICE(out, in, weight);
    CHECK_SAME_DTYPE(out->dtype(), in->dtype(), weight->dtype());
    CHECK_SAME_SHAPE(out->shape(), in->shape());
    CHECK_ARGUMENT(in->ndim() == 2 && weight->ndim() == 1 && weight->shape()[0] == in->shape()[1], "RmsNorm: shapes");
    ASSERT(out->isContiguous() && in->isContiguous() && weight->isContiguous(), "RmsNorm: tensors must be contiguous.");
    const size_t rows = in->shape()[0], d = in->shape()[1];
    LLAISYS_ON_DEVICE(out, cpu::rms_norm(out->dtype(), out->data(), in->data(), weight->data(), eps, rows, d),
                      kernels::rms_norm(stream, out->dtype(), out->data(), in->data(), weight->data(), eps, rows, d));
}

// out, in [seq, heads, d]; pos_ids [seq] int64 (reference: README.md:215-242)
void rope(tensor_t out, tensor_t in, tensor_t pos_ids, float theta) {
    CHECK_SAME_DEVICE(out, in, pos_ids);
    CHECK_SAME_DTYPE(out->dtype(), in->dtype());
    CHECK_SAME_SHAPE(out->shape(), in->shape());
    CHECK_ARGUMENT(pos_ids->dtype() == LLAISYS_DTYPE_I64, "ROPE: pos_ids must be int64");
    CHECK_ARGUMENT(in->ndim() == 3 && pos_ids->ndim() == 1 && pos_ids->shape()[0] == in->shape()[0], "ROPE: shapes");
    CHECK_ARGUMENT(in->shape()[2] % 2 == 0, "ROPE: head dimension must be even");
    ASSERT(out->isContiguous() && in->isContiguous() && pos_ids->isContiguous(), "ROPE: tensors must be contiguous.");
    const size_t seq = in->shape()[0], heads = in->shape()[1], d = in->shape()[2];
    LLAISYS_ON_DEVICE(out,
                      cpu::rope(out->dtype(), out->data(), in->data(), reinterpret_cast<const int64_t *>(pos_ids->data()),
                                theta, seq, heads, d),
                      kernels::rope(stream, out->dtype(), out->data(), in->data(),
                                    reinterpret_cast<const int64_t *>(pos_ids->data()), theta, seq, heads, d));
}

// out = up * gate / (1 + exp(-gate)) (reference: README.md:268-280)
void swiglu(tensor_t out, tensor_t gate, tensor_t up) {
    CHECK_SAME_DEVICE(out, gate, up);
    CHECK_SAME_DTYPE(out->dtype(), gate->dtype(), up->dtype());
    CHECK_SAME_SHAPE(out->shape(), gate->shape(), up->shape());
    ASSERT(out->isContiguous() && gate->isContiguous() && up->isContiguous(), "SwiGLU: tensors must be contiguous.");
    LLAISYS_ON_DEVICE(out, cpu::swiglu(out->dtype(), out->data(), gate->data(), up->data(), out->numel()),
                      kernels::swiglu(stream, out->dtype(), out->data(), gate->data(), up->data(), out->numel()));
}

} // namespace llaisys::ops
