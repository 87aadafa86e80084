// Host implementations of the same operations, for tensors and caches that live on LLAISYS_DEVICE_CPU.
// They are the library's CPU device backend (the reference keeps one beside every operator:
// src/ops/add/op.cpp:16-19, src/ops/add/cpu/add_cpu.cpp:7-32), selected only by the device type of the
// arguments -- never as a substitute for a missing or failing CUDA kernel.
#pragma once

#include "../kernels/args.hpp"

namespace llaisys::cpu {

void add(llaisysDataType_t dtype, void *c, const void *a, const void *b, size_t n);

void rearrange(size_t elem_size, size_t ndim, const size_t *shape, const ptrdiff_t *dst_strides,
               const ptrdiff_t *src_strides, void *dst, const void *src);

// Returns the OR of the kErr* bits (kernels/device_utils.cuh uses the same values) for rows it had to skip.
int paged_append(size_t elem_size, const kernels::KVView &kv, const void *k_rows, const void *v_rows,
                 const int32_t *seq_ids, const int32_t *positions, int32_t n_rows, int32_t max_blocks);
int paged_gather(size_t elem_size, const kernels::KVView &kv, int32_t seq_row, int32_t n_tokens, void *k_out,
                 void *v_out);
// Bias + rotary embedding + append over a packed projection qkv [n_rows, (nh + 2 nkvh) * d] (see kernels.hpp, K1b).
int paged_rope_append(llaisysDataType_t dtype, const kernels::KVView &kv, void *q_out, const void *qkv, const void *bias,
                      const int32_t *seq_ids, const int32_t *positions, int32_t n_rows, int32_t nh, float theta,
                      int32_t max_blocks);

// f32 accumulation, result rounded once to the tensor dtype ("compute in f32, store in T", the convention of
// the reference's only CPU kernel). Parallel over (query row, head) with OpenMP when built with it.
int attention(llaisysDataType_t dtype, const kernels::KVView &kv, const kernels::AttnBatch &batch, const void *q,
              float scale, const kernels::AttnOut &out);

void lse_merge(llaisysDataType_t dtype, void *out, const float *parts, int32_t n_parts, int32_t n_rows, int32_t d);

// ---- the remaining operators of the ABI (specs: reference README.md:157-302; oracles: reference test/ops/*.py).
// All arithmetic in f32 (f64 accumulation for the long dot products of linear), one rounding to the tensor dtype.

// Row-wise maximum: idx_out[r] (int64) = first index of the largest element of vals[r, :], val_out[r] = that element
// (val_out may be null).
void argmax_rows(llaisysDataType_t dtype, int64_t *idx_out, void *val_out, const void *vals, size_t rows, size_t n);
// out[i, :] = weight[index[i], :]
void embedding(size_t elem_size, void *out, const int64_t *index, const void *weight, size_t n, size_t d, size_t vocab);
// out[M, N] = in[M, K] . weight[N, K]^T (+ bias[N])
void linear(llaisysDataType_t dtype, void *out, const void *in, const void *weight, const void *bias, size_t m, size_t n,
            size_t k, bool accumulate = false); // accumulate: out += in . W^T
// out[r, :] = weight * in[r, :] / sqrt(mean(in[r, :]^2) + eps)
void rms_norm(llaisysDataType_t dtype, void *out, const void *in, const void *weight, float eps, size_t rows, size_t d);
// Rotary embedding with the half-split pairing (x[j], x[j + d/2]); angle = pos / theta^(2j/d) in f32.
void rope(llaisysDataType_t dtype, void *out, const void *in, const int64_t *pos, float theta, size_t seq, size_t heads,
          size_t d);
// out = up * gate / (1 + exp(-gate))
void swiglu(llaisysDataType_t dtype, void *out, const void *gate, const void *up, size_t n);
void swiglu_packed(llaisysDataType_t dtype, void *out, const void *gate_up, size_t rows, size_t di);

} // namespace llaisys::cpu
