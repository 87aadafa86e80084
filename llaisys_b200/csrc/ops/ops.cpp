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
    if (batch.const_q_len == 1) {
        size_t floats = 0, counters = 0;
        kernels::attention_decode_split_scratch(batch.n_seqs, batch.nh, view.nkvh, view.d, batch.max_kv_len, &floats,
                                                &counters);
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

// The remaining operators of the ABI are declared by the reference and left unimplemented there
// (src/ops/{argmax,embedding,linear,rms_norm,rope,swiglu}/op.cpp:4-6); they are outside the attention path.
void argmax(tensor_t, tensor_t, tensor_t) { TO_BE_IMPLEMENTED(); }
void embedding(tensor_t, tensor_t, tensor_t) { TO_BE_IMPLEMENTED(); }
void linear(tensor_t, tensor_t, tensor_t, tensor_t) { TO_BE_IMPLEMENTED(); }
void rms_norm(tensor_t, tensor_t, tensor_t, float) { TO_BE_IMPLEMENTED(); }
void rope(tensor_t, tensor_t, tensor_t, float) { TO_BE_IMPLEMENTED(); }
void swiglu(tensor_t, tensor_t, tensor_t) { TO_BE_IMPLEMENTED(); }

} // namespace llaisys::ops
