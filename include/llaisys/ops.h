/*
 * llaisys C ABI -- operators on tensor handles.
 *
 * Nine symbols, all returning void (reference: include/llaisys/ops.h:7-15, thunks in
 * src/llaisys/ops.cc:15-43). Outputs are pre-allocated by the caller; an operator never
 * allocates caller-visible memory and never synchronises: on NVIDIA it queues work on the
 * calling thread's runtime stream and returns.
 *
 * llaisysSelfAttention is the hot path of this library:
 *   attn_val[qlen, nh, dv] = causal_softmax(q[qlen, nh, d] . k[total, nkvh, d]^T * scale) . v[total, nkvh, dv]
 * where query i sees keys j <= i + (total - qlen) and query head h reads kv head h / (nh / nkvh)
 * (reference: test/ops/self_attention.py:11-28, README.md:244-266).
 */
#ifndef LLAISYS_OPS_H
#define LLAISYS_OPS_H

#include "tensor.h"

LLAISYS_EXTERN_C LLAISYS_API void llaisysAdd(llaisysTensor_t c, llaisysTensor_t a, llaisysTensor_t b);
LLAISYS_EXTERN_C LLAISYS_API void llaisysArgmax(llaisysTensor_t max_idx, llaisysTensor_t max_val, llaisysTensor_t vals);
LLAISYS_EXTERN_C LLAISYS_API void llaisysEmbedding(llaisysTensor_t out, llaisysTensor_t index, llaisysTensor_t weight);
LLAISYS_EXTERN_C LLAISYS_API void llaisysLinear(llaisysTensor_t out, llaisysTensor_t in, llaisysTensor_t weight,
                                                llaisysTensor_t bias);
/* New (no counterpart in the reference): out += in . weight^T, the sum rounded once -- the residual add of a decoder
 * block folded into its projection. Same shape rules and error behaviour as llaisysLinear. */
LLAISYS_EXTERN_C LLAISYS_API void llaisysLinearAccumulate(llaisysTensor_t out, llaisysTensor_t in, llaisysTensor_t weight);
/* New: which kernel serves decode-sized projections (at most 128 rows of 16-bit activations) on NVIDIA, process-wide.
 * 0 (default) = the hand-written tcgen05 weight-streaming kernel where it measured faster than cuBLAS (at most 16 rows
 * with K >= 4096), cuBLAS elsewhere; 1 = that kernel wherever its shape rules allow; 2 = always cuBLAS. Returns 0, or 1
 * for an unknown value (nothing changes). */
LLAISYS_EXTERN_C LLAISYS_API int llaisysSetLinearPolicy(int policy);
LLAISYS_EXTERN_C LLAISYS_API void llaisysRearrange(llaisysTensor_t out, llaisysTensor_t in);
LLAISYS_EXTERN_C LLAISYS_API void llaisysRmsNorm(llaisysTensor_t out, llaisysTensor_t in, llaisysTensor_t weight,
                                                 float eps);
LLAISYS_EXTERN_C LLAISYS_API void llaisysROPE(llaisysTensor_t out, llaisysTensor_t in, llaisysTensor_t pos_ids,
                                              float theta);
LLAISYS_EXTERN_C LLAISYS_API void llaisysSelfAttention(llaisysTensor_t attn_val, llaisysTensor_t q, llaisysTensor_t k,
                                                       llaisysTensor_t v, float scale);
LLAISYS_EXTERN_C LLAISYS_API void llaisysSwiGLU(llaisysTensor_t out, llaisysTensor_t gate, llaisysTensor_t up);

#endif /* LLAISYS_OPS_H */
