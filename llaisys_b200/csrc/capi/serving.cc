// extern "C" thunks of the batching engine (include/llaisys/serving.h).
#include "llaisys/serving.h"
#include "llaisys/paged_kv.h"

#include "../serve/engine.hpp"
#include "qwen2_handle.hpp"

namespace llaisys::kernels {
void set_last_error(const std::string &msg);
}

struct LlaisysEngine {
    llaisys::serve::Engine impl;
    LlaisysEngine(llaisys::models::Qwen2 &model, const llaisys::serve::EngineConfig &cfg) : impl(model, cfg) {}
};

static_assert(sizeof(LlaisysEngineEvent) == sizeof(llaisys::serve::Event), "event layouts must agree");

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
int null_handle() {
    llaisys::kernels::set_last_error("engine: null handle");
    return LLAISYS_E_INVALID;
}
} // namespace

extern "C" {

int llaisysEngineCreate(LlaisysEngine **engine_out, LlaisysQwen2Model *model, size_t max_batch, size_t max_tokens_per_step,
                        size_t prefill_chunk) {
    if (engine_out == nullptr || model == nullptr) {
        return null_handle();
    }
    return guarded([&] {
        llaisys::serve::EngineConfig cfg;
        cfg.max_batch = max_batch;
        cfg.max_tokens_per_step = max_tokens_per_step;
        cfg.prefill_chunk = prefill_chunk;
        *engine_out = new LlaisysEngine(model->impl, cfg);
    });
}
void llaisysEngineDestroy(LlaisysEngine *engine) { delete engine; }
int llaisysEngineSubmit(LlaisysEngine *engine, const int64_t *prompt, size_t n_prompt, size_t max_new_tokens,
                        int64_t end_token, int64_t *request_out) {
    if (engine == nullptr || request_out == nullptr) {
        return null_handle();
    }
    return guarded([&] { *request_out = engine->impl.submit(prompt, n_prompt, max_new_tokens, end_token); });
}
int llaisysEngineStep(LlaisysEngine *engine, LlaisysEngineEvent *events, size_t cap, size_t *n_events_out) {
    if (engine == nullptr || n_events_out == nullptr) {
        return null_handle();
    }
    return guarded(
        [&] { *n_events_out = engine->impl.step(reinterpret_cast<llaisys::serve::Event *>(events), cap); });
}
int llaisysEngineCancel(LlaisysEngine *engine, int64_t request) {
    if (engine == nullptr) {
        return null_handle();
    }
    return guarded([&] {
        if (!engine->impl.cancel(request)) {
            throw llaisys::kv::StatusError(LLAISYS_E_INVALID, "engine: no waiting or running request " + std::to_string(request));
        }
    });
}
size_t llaisysEngineNumWaiting(LlaisysEngine *engine) { return engine ? engine->impl.numWaiting() : 0; }
size_t llaisysEngineNumRunning(LlaisysEngine *engine) { return engine ? engine->impl.numRunning() : 0; }
size_t llaisysEngineCounter(LlaisysEngine *engine, int which) {
    if (engine == nullptr) {
        return 0;
    }
    switch (which) {
    case 0:
        return engine->impl.stepsRun();
    case 1:
        return engine->impl.promptTokensFromCache();
    case 2:
        return engine->impl.tokensComputed();
    default:
        return 0;
    }
}

} // extern "C"
