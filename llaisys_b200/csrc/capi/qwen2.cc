// extern "C" thunks of the Qwen2 model API. The four functions the reference declares keep its signatures (no status:
// failures print and abort like the rest of the legacy ABI); the new batched functions return status codes.
#include "llaisys/models/qwen2.h"
#include "llaisys/paged_kv.h"

#include "../models/qwen2.hpp"

#include <iostream>

#include "qwen2_handle.hpp"

namespace llaisys::kernels {
void set_last_error(const std::string &msg);
}

namespace {
template <typename F>
int guarded(F &&body) {
    try {
        body();
        return LLAISYS_OK;
    } catch (const llaisys::kv::StatusError &e) {
        llaisys::kernels::set_last_error(e.what());
        return e.code;
    } catch (const std::invalid_argument &e) {
        llaisys::kernels::set_last_error(e.what());
        return LLAISYS_E_INVALID;
    } catch (const std::exception &e) {
        llaisys::kernels::set_last_error(e.what());
        return LLAISYS_E_DEVICE;
    }
}
int null_model() {
    llaisys::kernels::set_last_error("qwen2: null model handle");
    return LLAISYS_E_INVALID;
}
} // namespace

extern "C" {

LlaisysQwen2Model *llaisysQwen2ModelCreate(const LlaisysQwen2Meta *meta, llaisysDeviceType_t device, int *device_ids,
                                           int ndevice) {
    if (meta == nullptr) {
        std::cerr << "[ERROR] llaisysQwen2ModelCreate: meta is null" << std::endl;
        return nullptr;
    }
    const int dev = (device_ids != nullptr && ndevice > 0) ? device_ids[0] : 0;
    LlaisysQwen2Model *model = nullptr;
    const int rc = guarded([&] { model = new LlaisysQwen2Model(*meta, device, dev); });
    if (rc != LLAISYS_OK) {
        std::cerr << "[ERROR] llaisysQwen2ModelCreate: " << llaisysGetLastError() << std::endl;
        return nullptr;
    }
    return model;
}

LlaisysQwen2Model *llaisysQwen2ModelCreateTP(const LlaisysQwen2Meta *meta, llaisysDeviceType_t device, int device_id,
                                             int tp_rank, int tp_world) {
    if (meta == nullptr) {
        std::cerr << "[ERROR] llaisysQwen2ModelCreateTP: meta is null" << std::endl;
        return nullptr;
    }
    LlaisysQwen2Model *model = nullptr;
    const int rc = guarded([&] { model = new LlaisysQwen2Model(*meta, device, device_id, tp_rank, tp_world); });
    if (rc != LLAISYS_OK) {
        std::cerr << "[ERROR] llaisysQwen2ModelCreateTP: " << llaisysGetLastError() << std::endl;
        return nullptr;
    }
    return model;
}

int llaisysNcclUniqueId(void *out_128_bytes) {
    return guarded([&] { llaisys::comm::ncclUniqueIdBytes(out_128_bytes); });
}

int llaisysQwen2ModelSetAllReduceNccl(LlaisysQwen2Model *model, const void *unique_id_128_bytes) {
    if (model == nullptr) {
        return null_model();
    }
    return guarded([&] {
        llaisys::core::context().setDevice(model->impl.deviceType(), model->impl.deviceId());
        model->impl.setCollective(
            llaisys::comm::Collective::nccl(unique_id_128_bytes, model->impl.tpRank(), model->impl.tpWorld()));
    });
}

int llaisysQwen2ModelSetAllReduceCallback(LlaisysQwen2Model *model, llaisysAllReduceFn fn, void *user) {
    if (model == nullptr) {
        return null_model();
    }
    return guarded([&] {
        model->impl.setCollective(llaisys::comm::Collective::callback(fn, user, model->impl.tpRank(), model->impl.tpWorld()));
    });
}

void llaisysQwen2ModelDestroy(LlaisysQwen2Model *model) { delete model; }

LlaisysQwen2Weights *llaisysQwen2ModelWeights(LlaisysQwen2Model *model) { return model ? model->impl.weights() : nullptr; }

int64_t llaisysQwen2ModelInfer(LlaisysQwen2Model *model, int64_t *token_ids, size_t ntoken) {
    // legacy convention: misuse throws through the C frame
    return model->impl.infer(token_ids, ntoken);
}

int llaisysQwen2ModelConfigureCache(LlaisysQwen2Model *model, size_t max_seqs, size_t max_tokens) {
    return model ? guarded([&] { model->impl.configureCache(max_seqs, max_tokens); }) : null_model();
}
int llaisysQwen2ModelSeqAdd(LlaisysQwen2Model *model, int32_t *seq_out) {
    if (model == nullptr || seq_out == nullptr) {
        return null_model();
    }
    return guarded([&] { *seq_out = model->impl.seqAdd(); });
}
int llaisysQwen2ModelSeqAddWithPrefix(LlaisysQwen2Model *model, const int64_t *tokens, size_t n, int32_t *seq_out,
                                      size_t *matched_out) {
    if (model == nullptr || seq_out == nullptr || matched_out == nullptr) {
        return null_model();
    }
    return guarded([&] { *seq_out = model->impl.seqAddWithPrefix(tokens, n, matched_out); });
}
int llaisysQwen2ModelSeqFree(LlaisysQwen2Model *model, int32_t seq) {
    return model ? guarded([&] { model->impl.seqFree(seq); }) : null_model();
}
int llaisysQwen2ModelReset(LlaisysQwen2Model *model) {
    return model ? guarded([&] { model->impl.reset(); }) : null_model();
}
int llaisysQwen2ModelStep(LlaisysQwen2Model *model, const int32_t *seq_ids, const int32_t *n_tokens, size_t n_seqs,
                          const int64_t *tokens, int64_t *next_out) {
    return model ? guarded([&] { model->impl.step(seq_ids, n_tokens, n_seqs, tokens, next_out); }) : null_model();
}
int llaisysQwen2ModelDecodeLoop(LlaisysQwen2Model *model, const int32_t *seq_ids, size_t n_seqs, const int64_t *first_tokens,
                                size_t n_steps, int64_t *tokens_out) {
    return model ? guarded([&] { model->impl.decodeLoop(seq_ids, n_seqs, first_tokens, n_steps, tokens_out); }) : null_model();
}
int llaisysQwen2ModelLastLogits(LlaisysQwen2Model *model, float *out_host, size_t capacity_floats) {
    return model ? guarded([&] { model->impl.lastLogits(out_host, capacity_floats); }) : null_model();
}
double llaisysQwen2ModelLastLoopMs(LlaisysQwen2Model *model) { return model ? model->impl.lastLoopMs() : 0.0; }

} // extern "C"
