// extern "C" thunks of the legacy ABI: tensors, operators, runtime (reference: src/llaisys/tensor.cc:5-96,
// src/llaisys/ops.cc:15-43, src/llaisys/runtime.cc:6-13). A handle is a heap object holding a shared_ptr, so
// views keep their storage alive and tensorDestroy only drops one reference.
#include "llaisys/ops.h"
#include "llaisys/runtime.h"
#include "llaisys/tensor.h"

#include "../device/runtime_api.hpp"
#include "handles.hpp"
#include "../ops/ops.hpp"
#ifdef ENABLE_NVIDIA_API
#include "../kernels/kernels.hpp"
#endif

#include <algorithm>


namespace {
llaisysTensor_t wrap(llaisys::tensor_t t) { return new LlaisysTensor{std::move(t)}; }
// A null handle stands for "no tensor" (the optional bias of llaisysLinear).
llaisys::tensor_t unwrap_optional(llaisysTensor_t h) { return h ? h->tensor : nullptr; }
} // namespace

extern "C" {

// ---- tensors ----
llaisysTensor_t tensorCreate(size_t *shape, size_t ndim, llaisysDataType_t dtype, llaisysDeviceType_t device_type,
                             int device_id) {
    return wrap(llaisys::Tensor::create(std::vector<size_t>(shape, shape + ndim), dtype, device_type, device_id));
}
void tensorDestroy(llaisysTensor_t tensor) { delete tensor; }
void *tensorGetData(llaisysTensor_t tensor) { return tensor->tensor->data(); }
size_t tensorGetNdim(llaisysTensor_t tensor) { return tensor->tensor->ndim(); }
void tensorGetShape(llaisysTensor_t tensor, size_t *shape) {
    const auto &s = tensor->tensor->shape();
    std::copy(s.begin(), s.end(), shape);
}
void tensorGetStrides(llaisysTensor_t tensor, ptrdiff_t *strides) {
    const auto &s = tensor->tensor->strides();
    std::copy(s.begin(), s.end(), strides);
}
llaisysDataType_t tensorGetDataType(llaisysTensor_t tensor) { return tensor->tensor->dtype(); }
llaisysDeviceType_t tensorGetDeviceType(llaisysTensor_t tensor) { return tensor->tensor->deviceType(); }
int tensorGetDeviceId(llaisysTensor_t tensor) { return tensor->tensor->deviceId(); }
void tensorDebug(llaisysTensor_t tensor) { tensor->tensor->debug(); }
uint8_t tensorIsContiguous(llaisysTensor_t tensor) { return tensor->tensor->isContiguous() ? 1 : 0; }
void tensorLoad(llaisysTensor_t tensor, const void *data) { tensor->tensor->load(data); }
llaisysTensor_t tensorView(llaisysTensor_t tensor, size_t *shape, size_t ndim) {
    return wrap(tensor->tensor->view(std::vector<size_t>(shape, shape + ndim)));
}
llaisysTensor_t tensorPermute(llaisysTensor_t tensor, size_t *order) {
    return wrap(tensor->tensor->permute(std::vector<size_t>(order, order + tensor->tensor->ndim())));
}
llaisysTensor_t tensorSlice(llaisysTensor_t tensor, size_t dim, size_t start, size_t end) {
    return wrap(tensor->tensor->slice(dim, start, end));
}

// ---- operators ----
void llaisysAdd(llaisysTensor_t c, llaisysTensor_t a, llaisysTensor_t b) {
    llaisys::ops::add(c->tensor, a->tensor, b->tensor);
}
void llaisysArgmax(llaisysTensor_t max_idx, llaisysTensor_t max_val, llaisysTensor_t vals) {
    llaisys::ops::argmax(max_idx->tensor, max_val->tensor, vals->tensor);
}
void llaisysEmbedding(llaisysTensor_t out, llaisysTensor_t index, llaisysTensor_t weight) {
    llaisys::ops::embedding(out->tensor, index->tensor, weight->tensor);
}
void llaisysLinear(llaisysTensor_t out, llaisysTensor_t in, llaisysTensor_t weight, llaisysTensor_t bias) {
    llaisys::ops::linear(out->tensor, in->tensor, weight->tensor, unwrap_optional(bias));
}
void llaisysLinearAccumulate(llaisysTensor_t out, llaisysTensor_t in, llaisysTensor_t weight) {
    llaisys::ops::linear_ex(out->tensor, in->tensor, weight->tensor, nullptr, true);
}
int llaisysSetLinearPolicy(int policy) {
#ifdef ENABLE_NVIDIA_API
    return llaisys::kernels::set_linear_policy(policy) ? 0 : 1;
#else
    return policy >= 0 && policy <= 2 ? 0 : 1; // CPU-only build: one kernel, nothing to choose
#endif
}
void llaisysRearrange(llaisysTensor_t out, llaisysTensor_t in) { llaisys::ops::rearrange(out->tensor, in->tensor); }
void llaisysRmsNorm(llaisysTensor_t out, llaisysTensor_t in, llaisysTensor_t weight, float eps) {
    llaisys::ops::rms_norm(out->tensor, in->tensor, weight->tensor, eps);
}
void llaisysROPE(llaisysTensor_t out, llaisysTensor_t in, llaisysTensor_t pos_ids, float theta) {
    llaisys::ops::rope(out->tensor, in->tensor, pos_ids->tensor, theta);
}
void llaisysSelfAttention(llaisysTensor_t attn_val, llaisysTensor_t q, llaisysTensor_t k, llaisysTensor_t v,
                          float scale) {
    llaisys::ops::self_attention(attn_val->tensor, q->tensor, k->tensor, v->tensor, scale);
}
void llaisysSwiGLU(llaisysTensor_t out, llaisysTensor_t gate, llaisysTensor_t up) {
    llaisys::ops::swiglu(out->tensor, gate->tensor, up->tensor);
}

// ---- runtime ----
const LlaisysRuntimeAPI *llaisysGetRuntimeAPI(llaisysDeviceType_t device_type) {
    return llaisys::device::getRuntimeAPI(device_type);
}
void llaisysSetContextRuntime(llaisysDeviceType_t device_type, int device_id) {
    llaisys::core::context().setDevice(device_type, device_id);
}
llaisysStream_t llaisysGetContextStream(void) { return llaisys::core::context().runtime().stream(); }

} // extern "C"
