/*
 * llaisys C ABI -- Qwen2 decoder model on top of the operators and the paged KV cache.
 *
 * The two structs and the first four functions are the reference's declaration (reference:
 * include/llaisys/models/qwen2.h:7-40), which it never implements (no qwen2 symbol is exported there). Weight
 * tensors are allocated by Create on the model's device; the caller fills them through the handles returned by
 * llaisysQwen2ModelWeights (tensorLoad) and must not destroy those handles. Linear weights are [out, in] row-major
 * (x . W^T), q/k/v projections carry biases, in_embed and out_embed are separate [voc, hs] tensors.
 *
 * llaisysQwen2ModelInfer keeps ONE implicit sequence: every call appends its ntoken tokens to that sequence's paged
 * cache (a multi-token call is a prefill chunk, a one-token call a decode step) and returns the greedy next token.
 * The functions below the line are new: batched sequences on the same cache, as a serving loop needs them.
 */
#ifndef LLAISYS_MODELS_QWEN2_H
#define LLAISYS_MODELS_QWEN2_H

#include "../tensor.h"

#ifdef __cplusplus
extern "C" {
#endif

struct LlaisysQwen2Meta {
    llaisysDataType_t dtype;
    size_t nlayer, hs, nh, nkvh, dh, di, maxseq, voc;
    float epsilon, theta;
    int64_t end_token;
};

struct LlaisysQwen2Weights {
    llaisysTensor_t in_embed;
    llaisysTensor_t out_embed;
    llaisysTensor_t out_norm_w;   /* model.norm.weight */
    llaisysTensor_t *attn_norm_w; /* input_layernorm.weight, one per layer (as all arrays below) */
    llaisysTensor_t *attn_q_w;
    llaisysTensor_t *attn_q_b;
    llaisysTensor_t *attn_k_w;
    llaisysTensor_t *attn_k_b;
    llaisysTensor_t *attn_v_w;
    llaisysTensor_t *attn_v_b;
    llaisysTensor_t *attn_o_w;
    llaisysTensor_t *mlp_norm_w; /* post_attention_layernorm.weight */
    llaisysTensor_t *mlp_gate_w;
    llaisysTensor_t *mlp_up_w;
    llaisysTensor_t *mlp_down_w;
};

struct LlaisysQwen2Model;

/* device_ids[0] is used (one process drives one GPU; sequences are sharded across processes). */
LLAISYS_API struct LlaisysQwen2Model *llaisysQwen2ModelCreate(const struct LlaisysQwen2Meta *meta,
                                                              llaisysDeviceType_t device, int *device_ids, int ndevice);
LLAISYS_API void llaisysQwen2ModelDestroy(struct LlaisysQwen2Model *model);
LLAISYS_API struct LlaisysQwen2Weights *llaisysQwen2ModelWeights(struct LlaisysQwen2Model *model);
LLAISYS_API int64_t llaisysQwen2ModelInfer(struct LlaisysQwen2Model *model, int64_t *token_ids, size_t ntoken);

/* ---- new: batched sequences (status codes as in paged_kv.h; no counterpart in the reference) -------------------- */

/* Sizes the paged cache: at most max_seqs live sequences of at most max_tokens tokens each (page size 16). Must be
 * called before the first batched call; llaisysQwen2ModelInfer sizes a one-sequence cache of meta.maxseq by itself. */
LLAISYS_API int llaisysQwen2ModelConfigureCache(struct LlaisysQwen2Model *model, size_t max_seqs, size_t max_tokens);
LLAISYS_API int llaisysQwen2ModelSeqAdd(struct LlaisysQwen2Model *model, int32_t *seq_out);
/* As SeqAdd, but the new sequence starts from cached K/V: the model publishes the full pages of every sequence it runs
 * under their token ids, and this call attaches the pages matching the longest whole-page prefix of tokens[0, n) that
 * still leaves one token to run. *matched_out = tokens covered; feed tokens[*matched_out, n) to the first Step. */
LLAISYS_API int llaisysQwen2ModelSeqAddWithPrefix(struct LlaisysQwen2Model *model, const int64_t *tokens, size_t n,
                                                  int32_t *seq_out, size_t *matched_out);
LLAISYS_API int llaisysQwen2ModelSeqFree(struct LlaisysQwen2Model *model, int32_t seq);
/* Forgets the implicit sequence of llaisysQwen2ModelInfer. */
LLAISYS_API int llaisysQwen2ModelReset(struct LlaisysQwen2Model *model);
/* Appends n_tokens[i] new tokens (tokens, packed back to back, host int64) to sequence seq_ids[i] and writes the greedy
 * next token of every sequence to next_out[n_seqs] (host). Any mix of chunk lengths >= 1. */
LLAISYS_API int llaisysQwen2ModelStep(struct LlaisysQwen2Model *model, const int32_t *seq_ids, const int32_t *n_tokens,
                                      size_t n_seqs, const int64_t *tokens, int64_t *next_out);
/* n_steps greedy decode steps for the given sequences, starting from first_tokens[n_seqs] (the tokens returned by the
 * previous step): the loop stays on the device (token feedback, positions and lengths advance there; on NVIDIA the step
 * is captured once as a CUDA graph and replayed). tokens_out is host int64 [n_steps][n_seqs]. */
LLAISYS_API int llaisysQwen2ModelDecodeLoop(struct LlaisysQwen2Model *model, const int32_t *seq_ids, size_t n_seqs,
                                            const int64_t *first_tokens, size_t n_steps, int64_t *tokens_out);
/* Copies the logits of the most recent step, float32 [n_seqs of that step][voc], to host memory. */
LLAISYS_API int llaisysQwen2ModelLastLogits(struct LlaisysQwen2Model *model, float *out_host, size_t capacity_floats);
/* Average milliseconds of device time per decode step of the last llaisysQwen2ModelDecodeLoop: CUDA events on the
 * launch stream around the graph replays (the first step runs eagerly, to size scratch, and is not timed); wall clock
 * over all steps on CPU. 0 when the loop had a single step. */
LLAISYS_API double llaisysQwen2ModelLastLoopMs(struct LlaisysQwen2Model *model);

/* ---- new: tensor parallelism (no counterpart in the reference, which names it as future work: README.md:426-427) -- */

/* As llaisysQwen2ModelCreate, for rank tp_rank of tp_world processes that share ONE model (one process per GPU). meta
 * holds the whole model's dimensions; tp_world must divide nkvh, nh and di. The rank holds query heads
 * [r nh/W, (r+1) nh/W) with their KV heads and rows [r di/W, (r+1) di/W) of the MLP: the weight handles have the
 * sharded shapes -- attn_q_w [nh/W * dh, hs], attn_k_w / attn_v_w [nkvh/W * dh, hs] and their biases, attn_o_w
 * [hs, nh/W * dh], mlp_gate_w / mlp_up_w [di/W, hs], mlp_down_w [hs, di/W] -- and take the matching slices of the
 * checkpoint; embeddings, norms and out_embed are replicated. Every rank must make the same calls with the same tokens;
 * every rank gets the same logits and tokens. Two all-reduces of [tokens, hs] per layer (after the output and down
 * projections) run through the collective set below. */
LLAISYS_API struct LlaisysQwen2Model *llaisysQwen2ModelCreateTP(const struct LlaisysQwen2Meta *meta,
                                                                llaisysDeviceType_t device, int device_id, int tp_rank,
                                                                int tp_world);
/* NCCL all-reduce on the model's stream. unique_id: the 128 bytes rank 0 got from llaisysNcclUniqueId and sent to the
 * other ranks over any host channel. Collective call: every rank of the group must make it. */
LLAISYS_API int llaisysNcclUniqueId(void *out_128_bytes);
LLAISYS_API int llaisysQwen2ModelSetAllReduceNccl(struct LlaisysQwen2Model *model, const void *unique_id_128_bytes);
/* Host all-reduce for CPU models: fn sums `count` elements of `dtype` (llaisysDataType_t) at `buf` in place over the
 * ranks and returns 0. */
typedef int (*llaisysAllReduceFn)(void *buf, size_t count, int dtype, void *user);
LLAISYS_API int llaisysQwen2ModelSetAllReduceCallback(struct LlaisysQwen2Model *model, llaisysAllReduceFn fn, void *user);

#ifdef __cplusplus
}
#endif
#endif /* LLAISYS_MODELS_QWEN2_H */
