/*
 * llaisys C ABI -- iteration-level ("continuous") batching engine over a Qwen2 model and its paged KV cache.
 *
 * New: the reference describes a multi-user service with a request queue, continuous batching and a KV-cache pool with
 * prefix matching as future work (reference: README.md:415-424) and has no code for it. Status codes as in paged_kv.h.
 * An engine belongs to the thread that drives it. It borrows the model: destroy the engine first; if the model goes
 * first the engine drops its requests and every later call on it returns LLAISYS_E_INVALID (destroying it stays safe).
 */
#ifndef LLAISYS_SERVING_H
#define LLAISYS_SERVING_H

#include "models/qwen2.h"

#ifdef __cplusplus
extern "C" {
#endif

struct LlaisysEngine;

struct LlaisysEngineEvent {
    int64_t request;  /* id returned by llaisysEngineSubmit */
    int64_t token;    /* token generated for the request in this step */
    int32_t finished; /* 1 = last token of the request (length limit or end token) */
    int32_t reserved;
};

/* max_batch requests per step; at most max_tokens_per_step tokens per step (one per decoding request first, prompt
 * chunks of at most prefill_chunk tokens per request with the rest). llaisysQwen2ModelConfigureCache must have sized
 * the model's cache: its max_seqs bounds the live requests, its pages bound what can be admitted. */
LLAISYS_API int llaisysEngineCreate(struct LlaisysEngine **engine_out, struct LlaisysQwen2Model *model, size_t max_batch,
                                    size_t max_tokens_per_step, size_t prefill_chunk);
LLAISYS_API void llaisysEngineDestroy(struct LlaisysEngine *engine);
/* Queues a request (first come, first served). end_token < 0 = the model's. A request is admitted to the running set
 * once the pool holds pages for its prompt and all it may generate; its prompt first reuses whole pages that earlier
 * requests with the same beginning left in the prefix cache. */
LLAISYS_API int llaisysEngineSubmit(struct LlaisysEngine *engine, const int64_t *prompt, size_t n_prompt,
                                    size_t max_new_tokens, int64_t end_token, int64_t *request_out);
/* One iteration: admits what fits, runs one batched model step, writes one event per request that produced a token
 * (at most max_batch; `cap` must be at least that), frees finished requests. *n_events_out = 0 with nothing to do. */
LLAISYS_API int llaisysEngineStep(struct LlaisysEngine *engine, struct LlaisysEngineEvent *events, size_t cap,
                                  size_t *n_events_out);
/* Drops a waiting or running request; LLAISYS_E_INVALID if the id is unknown or already finished. */
LLAISYS_API int llaisysEngineCancel(struct LlaisysEngine *engine, int64_t request);
LLAISYS_API size_t llaisysEngineNumWaiting(struct LlaisysEngine *engine);
LLAISYS_API size_t llaisysEngineNumRunning(struct LlaisysEngine *engine);
/* Counters since creation: which = 0 steps run, 1 prompt tokens taken from the prefix cache, 2 tokens computed. */
LLAISYS_API size_t llaisysEngineCounter(struct LlaisysEngine *engine, int which);

#ifdef __cplusplus
}
#endif
#endif /* LLAISYS_SERVING_H */
