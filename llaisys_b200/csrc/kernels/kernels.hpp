// Host-callable launchers of every CUDA kernel in the library. Each launcher queues work on `stream` and
// returns; none allocates, synchronises or touches host copies of the data. Launchers that return int give
// 0 when work was queued and a negative value when they have no kernel for the shape (the caller then picks
// another launcher); launch failures throw.
#pragma once

#include "args.hpp"

namespace llaisys::kernels {

// Queues a memset of `bytes` zero bytes.
void fill_zero(stream_t stream, void *ptr, size_t bytes);
// The address under which kernels of the current device can read a host buffer directly: non-null only for page-locked
// host memory that is mapped into the device's address space (what cudaHostAlloc / cudaMallocHost and torch's pinned
// tensors give); null for pageable memory, for device memory and on any error.
// All `bytes` bytes from host_ptr on must lie inside one such allocation.
const void *mapped_host_alias(const void *host_ptr, size_t bytes);
// Up to three plain copies (each a 16-byte aligned multiple of 16 bytes) done by ONE kernel launch: for small blocks in
// mapped host memory, where a kernel's loads start sooner than a copy-engine transfer is set up.
void small_copies(stream_t stream, const void *const *src, void *const *dst, const size_t *bytes, int n);

// c = a + b over n contiguous elements of F32 / F16 / BF16 (arithmetic in f32).
void add(stream_t stream, llaisysDataType_t dtype, void *c, const void *a, const void *b, size_t n);

// Strided copy dst[idx] = src[idx] for every index of `shape` (ndim <= 8), elements of elem_size bytes.
void rearrange(stream_t stream, size_t elem_size, size_t ndim, const size_t *shape, const ptrdiff_t *dst_strides,
               const ptrdiff_t *src_strides, void *dst, const void *src);

// The operators around the attention path (specs: reference README.md:157-302). HBM-bound single-pass kernels; linear is
// a cuBLAS GEMM (f32 accumulation) followed by the bias add.
void argmax_rows(stream_t stream, llaisysDataType_t dtype, int64_t *idx_out, void *val_out, const void *vals, size_t rows,
                 size_t n);
void embedding(stream_t stream, size_t elem_size, void *out, const int64_t *index, const void *weight, size_t n, size_t d,
               size_t vocab);
// accumulate: out += in . W^T (the residual add of a decoder block folded into the projection; one rounding of the sum)
void linear(stream_t stream, llaisysDataType_t dtype, void *out, const void *in, const void *weight, const void *bias,
            size_t m, size_t n, size_t k, bool accumulate = false);
// K6: the tcgen05 weight-streaming kernel behind linear() for at most 128 rows of 16-bit activations (K a multiple of 64,
// N a multiple of 64, not vocabulary-sized). False = shape not covered, nothing launched. overlap: programmatic launch
// (the weight stream starts under the previous kernel's tail). linear_tc_status synchronises the stream and returns (and
// clears) the kernel's error word: 0, or 16 when a bounded wait ran out.
// 0 = the streaming kernel where it measured faster (default), 1 = wherever it applies, 2 = never. False: unknown value.
bool set_linear_policy(int policy);
bool linear_tc(stream_t stream, llaisysDataType_t dtype, void *out, const void *in, const void *weight, size_t m, size_t n,
               size_t k, bool accumulate, bool overlap);
int linear_tc_status(stream_t stream);
// out[r, i] = up * silu(gate) with gate = gu[r, i], up = gu[r, di + i]: the activation on a packed gate|up projection.
void swiglu_packed(stream_t stream, llaisysDataType_t dtype, void *out, const void *gate_up, size_t rows, size_t di);
// Row-wise argmax with every row split over several CTAs (a vocabulary-sized row on one CTA leaves the GPU idle).
// scratch: 12 * rows bytes, zero before the first call; the kernel leaves it zero again.
void argmax_rows_split(stream_t stream, llaisysDataType_t dtype, int64_t *idx_out, const void *vals, size_t rows, size_t n,
                       void *scratch);
void bias_add(stream_t stream, llaisysDataType_t dtype, void *out, const void *bias, size_t rows, size_t n);
void rms_norm(stream_t stream, llaisysDataType_t dtype, void *out, const void *in, const void *weight, float eps, size_t rows,
              size_t d);
void rope(stream_t stream, llaisysDataType_t dtype, void *out, const void *in, const int64_t *pos, float theta, size_t seq,
          size_t heads, size_t d);
void swiglu(stream_t stream, llaisysDataType_t dtype, void *out, const void *gate, const void *up, size_t n);

// Device-resident decode loop support: state hand-over between steps, CUDA graph capture / replay, event timing.
void advance_decode_state(stream_t stream, int64_t *tokens, const int64_t *next, int64_t *pos64, int32_t *pos32,
                          int32_t *kv_lens, int64_t *log, int32_t *step_counter, int n);
void graph_capture_begin(stream_t stream);
void *graph_capture_end(stream_t stream); // instantiated executable graph
void graph_launch(void *exec, stream_t stream);
void graph_destroy(void *exec);
void *event_create();
void event_record(void *event, stream_t stream);
float event_elapsed_ms(void *start, void *stop); // synchronises on `stop`
void event_destroy(void *event);

// K1: row i of k_rows / v_rows [n_rows, nkvh, d] -> token positions[i] of the sequence in table row seq_ids[i].
// 16-byte vector copies; a row whose block or page is out of range is skipped and flagged. side_src / side_dst: an
// optional plain copy of side_bytes (a multiple of 16) done by the same launch.
void paged_append(stream_t stream, size_t elem_size, const KVView &kv, const void *k_rows, const void *v_rows,
                  const int32_t *seq_ids, const int32_t *positions, int32_t n_rows, int32_t max_blocks,
                  int32_t *error_flag, const void *side_src = nullptr, void *side_dst = nullptr, size_t side_bytes = 0);

// K1b: bias + rotary embedding + append in one pass over the packed projection qkv [n_rows, (nh + 2 nkvh) * d]: rotated q
// -> q_out [n_rows, nh, d]; rotated k and plain v -> their page slots (same addressing and flags as K1).
void paged_rope_append(stream_t stream, llaisysDataType_t dtype, const KVView &kv, void *q_out, const void *qkv,
                       const void *bias, const int32_t *seq_ids, const int32_t *positions, int32_t n_rows, int32_t nh,
                       float theta, int32_t max_blocks, int32_t *error_flag);

// K5: tokens [0, n_tokens) of table row seq_row -> k_out, v_out [n_tokens, nkvh, d].
void paged_gather(stream_t stream, size_t elem_size, const KVView &kv, int32_t seq_row, int32_t n_tokens,
                  void *k_out, void *v_out, int32_t *error_flag);

// Any dtype, head_dim <= 256, any GQA ratio, any page size: one CTA per (query row, query head), online
// softmax in f32. The correctness baseline for the specialised kernels and the kernel behind the legacy
// operator for shapes they do not cover.
void attention_generic(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                       const void *q, float scale, const AttnOut &out, int32_t *error_flag);

// K2 (+ fused K3): split-KV flash decoding for 16-bit K/V, head_dim 128, page size 16, GQA group <= 8,
// one query per sequence. Returns -1 if the shape is not covered.
int attention_decode_split(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                           const void *q, float scale, const AttnOut &out, const AttnScratch &scratch);
// Scratch the split-KV decode needs for a batch of n_seqs sequences of at most max_kv_len tokens.
void attention_decode_split_scratch(int32_t n_seqs, int32_t nh, int32_t nkvh, int32_t d, int32_t max_kv_len,
                                    size_t *partials_floats, size_t *counters_len);

// Number of persistent CTAs the split-KV decode kernels launch for a batch (two per SM, fewer for tiny batches).
int decode_grid_size(int32_t n_seqs, int32_t nkvh, int32_t max_kv_len);

// TMA edition of K2 + K3 for page pools that carry a tensor map (KVView::tma_desc). Same contract and scratch
// as attention_decode_split. k_new / v_new (both or neither; [n_seqs, nkvh, 128], 16-byte aligned): fused step -- row i
// is also appended as token kv_lens[i] - 1 of sequence i by the same launch. Returns -1 and sets *why (a static string)
// if the view or shape is not covered; nothing is queued then.
int attention_decode_tma(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                         const void *q, float scale, const AttnOut &out, const AttnScratch &scratch,
                         const void *k_new = nullptr, const void *v_new = nullptr, const char **why = nullptr);
// Encodes the tensor map over a 16-bit page pool (head_dim 128, page 16) starting at pool_base into out_128_bytes
// (host memory): total_rows rows of 128 elements, nkvh of them per (page, K|V) block of 16 slots each. Returns -1
// when the driver cannot provide one (the cp.async kernel is used then).
int make_kv_tensor_map(void *out_128_bytes, void *pool_base, uint64_t total_rows, uint32_t nkvh, llaisysDataType_t dtype);

// K4: chunked-prefill attention on tcgen05 for page pools that carry the half-tile tensor map
// (KVView::tma_tile_desc): 16-bit K/V, head_dim 128, page 16, ragged causal chunks (batch.q_starts). Returns -1 if
// the view or shape is not covered, or the scratch is smaller than attention_prefill_tc_scratch asks for (partial
// results of tiles that are split over CTAs, and their arrival counters, which must be zero between launches).
int attention_prefill_tc(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                         const void *q, float scale, const AttnOut &out, const AttnScratch &scratch);
void attention_prefill_tc_scratch(size_t *floats, size_t *counters);
// Two maps, 128 bytes each: the half-tile map (K) and the whole-tile-as-two-halves map (V).
int make_kv_tile_tensor_map(void *out_256_bytes, void *pool_base, uint64_t total_rows, uint32_t nkvh,
                            llaisysDataType_t dtype);

// K3: out[r, :] = sum_p w_p o_p[r, :] / sum_p w_p, w_p = l_p exp(m_p - max_p m_p), over n_parts partials laid out
// float [n_parts][n_rows][d + 2].
void lse_merge(stream_t stream, llaisysDataType_t dtype, void *out, const float *parts, int32_t n_parts,
               int32_t n_rows, int32_t d);

} // namespace llaisys::kernels
