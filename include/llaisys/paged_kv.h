/*
 * llaisys C ABI -- paged KV cache and the attention kernels that read it.
 *
 * NEW SURFACE. The reference has no KV cache: its self-attention operator takes whole
 * contiguous K/V tensors (reference: src/ops/self_attention/op.hpp:6, README.md:244-266) and
 * names a KV cache / KV-cache pool only as future work (reference: README.md:316, :412, :424).
 * These entry points are what the reference's FFI would bind for that work. They follow the
 * reference's conventions where it has any (C linkage, llaisys prefix, enums from llaisys.h,
 * async on the calling thread's runtime stream, caller-allocated outputs) and differ in one:
 * every function returns a status code and never throws across the ABI.
 *
 * Arithmetic contract of the attention calls is the reference's definition of self-attention
 * (reference: test/ops/self_attention.py:11-28) applied to the K/V rows a sequence holds in the
 * cache: gathering a sequence's pages to contiguous [len, nkvh, d] tensors and calling
 * llaisysSelfAttention must give the same result within rounding.
 *
 * Memory layout of the pool (one allocation, made once at create):
 *     pool[layer][page][2 (K=0, V=1)][nkvh][page_size][head_dim]      row-major, `dtype` elements
 * so a (page, K-or-V, kv-head) tile is page_size*head_dim contiguous elements (4 KiB for bf16,
 * page 16, d 128) and token `pos` of a sequence lives in slot  table[seq][pos / page_size] * page_size
 * + pos % page_size.
 *
 * Pointer conventions: `*_dev` arguments and all bulk tensors (q, out, k_rows, ...) are addresses
 * in the cache's device memory (host memory for a CPU cache); small index arrays WITHOUT the
 * suffix are host arrays that the call validates and stages itself.
 */
#ifndef LLAISYS_PAGED_KV_H
#define LLAISYS_PAGED_KV_H

#include "../llaisys.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------------------- */
#define LLAISYS_OK 0
#define LLAISYS_E_INVALID 1     /* bad argument, shape, dtype or sequence state            */
#define LLAISYS_E_NO_PAGES 2    /* the free list cannot cover the request (nothing changed) */
#define LLAISYS_E_NO_SEQ 3      /* unknown / freed sequence id, or max_seqs reached         */
#define LLAISYS_E_DEVICE 4      /* the device runtime reported an error                     */
#define LLAISYS_E_UNSUPPORTED 5 /* no kernel for this dtype / shape on this device          */
#define LLAISYS_E_KERNEL 6      /* a kernel flagged bad metadata instead of faulting        */

/* Text of the calling thread's most recent non-OK status ("" if none). */
LLAISYS_API const char *llaisysGetLastError(void);

/* ---- which kernel served an attention call ------------------------------------------------ */
/* The library picks the kernel from the call's shape alone and says which one it queued. Pools of 16-bit data with
 * head_dim 128, 16-token pages and at most 8 query heads per kv head are served by the TMA decode kernel and the
 * tcgen05 chunk kernel and by nothing else: a call of that shape they cannot take (misaligned buffers, ...) returns
 * LLAISYS_E_UNSUPPORTED with the reason in llaisysGetLastError; it is never re-routed to the generic kernel. */
#define LLAISYS_KERNEL_NONE 0
#define LLAISYS_KERNEL_CPU 1              /* the host loops of a CPU cache / CPU tensors                          */
#define LLAISYS_KERNEL_GENERIC 2          /* CUDA, any dtype / head_dim / page size: one CTA per (query, head)    */
#define LLAISYS_KERNEL_DECODE_TMA 3       /* split-KV flash decoding over a page pool, TMA copy pipeline          */
#define LLAISYS_KERNEL_DECODE_TMA_FUSED 4 /* the same launch also appends the step's new K/V rows                 */
#define LLAISYS_KERNEL_DECODE_CP_ASYNC 5  /* split-KV flash decoding over plain K/V tensors (legacy operator)     */
#define LLAISYS_KERNEL_PREFILL_TC 6       /* causal chunk attention on tcgen05 tensor cores                       */
/* Kernel of the calling thread's most recent attention call: any cache, or llaisysSelfAttention. */
LLAISYS_API int llaisysLastAttentionKernel(void);

typedef struct LlaisysPagedKV *llaisysPagedKV_t;

/* ---- lifetime ------------------------------------------------------------------------ */

/* Allocates the page pool, block tables and the attention kernels' workspace on (device_type, device_id): everything
 * a data-path call with device index arrays will ever need (for 16-bit, head_dim 128, page 16 pools on NVIDIA about
 * 40 MiB beside the pool), so those calls never allocate and CUDA graphs captured over them stay valid.
 * max_seqs bounds live sequences; max_pages_per_seq bounds one sequence's block table.
 * dtype is F32, F16 or BF16. */
LLAISYS_API int llaisysPagedKVCreate(llaisysPagedKV_t *kv_out, llaisysDeviceType_t device_type, int device_id,
                                     llaisysDataType_t dtype, size_t nlayer, size_t num_pages, size_t page_size,
                                     size_t nkvh, size_t head_dim, size_t max_seqs, size_t max_pages_per_seq);
LLAISYS_API int llaisysPagedKVDestroy(llaisysPagedKV_t kv);

/* ---- block manager (host only; no device work) ---------------------------------------- */

/* New empty sequence; its id (0 <= id < max_seqs) is written to *seq_out. */
LLAISYS_API int llaisysPagedKVSeqAdd(llaisysPagedKV_t kv, int32_t *seq_out);
/* Grows the sequence's capacity to at least n_tokens by popping pages off the free list.
 * All-or-nothing: on LLAISYS_E_NO_PAGES the sequence and the free list are unchanged. */
LLAISYS_API int llaisysPagedKVSeqReserve(llaisysPagedKV_t kv, int32_t seq, size_t n_tokens);
/* Appends the given physical pages (each must be free) to the sequence's block table. */
LLAISYS_API int llaisysPagedKVSeqAssignPages(llaisysPagedKV_t kv, int32_t seq, const int32_t *pages, size_t n_pages);
/* Returns every page of the sequence to the free list and retires the id. */
LLAISYS_API int llaisysPagedKVSeqFree(llaisysPagedKV_t kv, int32_t seq);

LLAISYS_API size_t llaisysPagedKVNumFreePages(llaisysPagedKV_t kv);
LLAISYS_API size_t llaisysPagedKVNumSeqs(llaisysPagedKV_t kv);
/* Pages held by a sequence, or -1 for an unknown id. */
LLAISYS_API int64_t llaisysPagedKVSeqNumPages(llaisysPagedKV_t kv, int32_t seq);
/* Copies up to `cap` block-table entries of the sequence into pages_out. */
LLAISYS_API int llaisysPagedKVSeqPages(llaisysPagedKV_t kv, int32_t seq, int32_t *pages_out, size_t cap);

/* ---- prefix sharing (block manager, host only) -------------------------------------------- */
/* Pages are reference-counted. A sequence's whole pages can be published under the chain of their token ids and found
 * again by later sequences that start with the same tokens (the KV-cache pool with prefix matching the reference's
 * README.md:412 and :424 ask for); shared pages are never written again, because a sequence only appends behind the
 * tokens it holds. When the last holder of a published page goes, the page stays findable ("cached") until the pool
 * needs it; cached pages count as free and the one released longest ago is reused first. */

/* Registers the full pages of the sequence under tokens[0, n_tokens): the ids of the tokens whose K/V it holds. */
LLAISYS_API int llaisysPagedKVSeqPublish(llaisysPagedKV_t kv, int32_t seq, const int64_t *tokens, size_t n_tokens);
/* Attaches to an EMPTY sequence the published pages matching the longest whole-page prefix of tokens[0, n_tokens);
 * *matched_out = tokens covered (a multiple of the page size). The caller appends from position *matched_out. */
LLAISYS_API int llaisysPagedKVSeqMatchPrefix(llaisysPagedKV_t kv, int32_t seq, const int64_t *tokens, size_t n_tokens,
                                             size_t *matched_out);
/* New sequence sharing the parent's first n_tokens: whole pages by reference, a partial last page by copy (every
 * layer; the copies are queued on the calling thread's stream behind the work already queued there). */
LLAISYS_API int llaisysPagedKVSeqFork(llaisysPagedKV_t kv, int32_t parent, size_t n_tokens, int32_t *child_out);
/* Number of sequences holding the page (0 = free or cached), -1 for a bad handle or page. */
LLAISYS_API int llaisysPagedKVPageRefCount(llaisysPagedKV_t kv, int32_t page);
/* Cached pages: released by every holder, still findable by prefix (included in llaisysPagedKVNumFreePages). */
LLAISYS_API size_t llaisysPagedKVNumCachedPages(llaisysPagedKV_t kv);

/* ---- device-side views ----------------------------------------------------------------- */

LLAISYS_API void *llaisysPagedKVPoolData(llaisysPagedKV_t kv, size_t layer); /* pool[layer]          */
LLAISYS_API size_t llaisysPagedKVLayerBytes(llaisysPagedKV_t kv);
/* int32 table[max_seqs][max_pages_per_seq] in device memory. Rows changed by the block manager
 * reach the device at the next data-path call, or at llaisysPagedKVFlush. */
LLAISYS_API const int32_t *llaisysPagedKVBlockTableData(llaisysPagedKV_t kv);
LLAISYS_API int llaisysPagedKVFlush(llaisysPagedKV_t kv);
/* Opt-in (default off), meant for decode loops (append one row per sequence, decode, repeat): launch the append and
 * decode kernels with programmatic stream serialisation, so that a decode kernel's set-up and its copies of OLDER
 * pages overlap the tail of the kernels before it on the stream. A decode kernel touches q, each sequence's LAST
 * page, scratch and outputs only after the kernel directly before it has completed, and lets its own successor start
 * only after that; the append kernel waits for its predecessor before doing anything. Contract while overlap is on:
 *   - the kernel directly before a decode call on the stream writes K/V only into the last two token slots of each
 *     sequence (positions kv_len - 2 and kv_len - 1 by the kv_lens of that decode call) -- true for a one-row-per-
 *     sequence append and for the one-launch decode step of the token before; after a multi-page append (a prefill
 *     chunk) put any non-overlapping kernel, a copy or a synchronisation before the first decode call;
 *   - index arrays and block-table rows passed to a call were written before that directly preceding kernel started
 *     (true for host-array calls, whose staging copies break the chain, and for device arrays prepared per batch).
 * The chunked-prefill kernel takes part too: it reads its index arrays, sums the work and sets up its on-chip state
 * before waiting, and touches q, K/V, workspace and outputs only after the kernel directly before it has completed. */
LLAISYS_API int llaisysPagedKVSetLaunchOverlap(llaisysPagedKV_t kv, int enable);
/* LLAISYS_KERNEL_* of this cache's most recent attention call (-1 for a null handle). */
LLAISYS_API int llaisysPagedKVLastKernel(llaisysPagedKV_t kv);
/* Synchronises the cache's stream and reports LLAISYS_E_KERNEL if any kernel since the last
 * check met an out-of-range page or position (the kernel skips such an access). */
LLAISYS_API int llaisysPagedKVCheck(llaisysPagedKV_t kv);

/* ---- data path, host index arrays ------------------------------------------------------ */

/* Scatters n_rows new K/V rows into the pages: row i goes to token `positions[i]` of sequence
 * `seq_ids[i]`. k_rows / v_rows are [n_rows, nkvh, head_dim]. Bit-exact copy. */
LLAISYS_API int llaisysPagedKVAppend(llaisysPagedKV_t kv, size_t layer, const void *k_rows, const void *v_rows,
                                     const int32_t *seq_ids, const int32_t *positions, size_t n_rows);
/* Inverse of append for one sequence: tokens [0, n_tokens) -> k_out, v_out [n_tokens, nkvh, head_dim]. */
LLAISYS_API int llaisysPagedKVGather(llaisysPagedKV_t kv, size_t layer, int32_t seq, size_t n_tokens, void *k_out,
                                     void *v_out);

/* One query token per sequence: out, q are [n_seqs, nh, head_dim]; sequence i attends to its first
 * kv_lens[i] tokens (all visible: the single query is the newest token). */
LLAISYS_API int llaisysPagedAttentionDecode(llaisysPagedKV_t kv, size_t layer, void *out, const void *q,
                                            const int32_t *seq_ids, const int32_t *kv_lens, size_t n_seqs, size_t nh,
                                            float scale);
/* Ragged chunks: q, out are [sum(q_lens), nh, head_dim], sequences back to back. Query t of sequence i
 * (0 <= t < q_lens[i]) sees keys j <= t + (kv_lens[i] - q_lens[i]); kv_lens counts the chunk itself,
 * which the caller has already appended. */
LLAISYS_API int llaisysPagedAttentionPrefill(llaisysPagedKV_t kv, size_t layer, void *out, const void *q,
                                             const int32_t *seq_ids, const int32_t *q_lens, const int32_t *kv_lens,
                                             size_t n_seqs, size_t nh, float scale);
/* Decode that stops before normalising across devices: part is float [n_seqs, nh, head_dim + 2] holding,
 * per (sequence, head), the locally normalised output o[0..d), then m = max scaled score and
 * l = sum exp(score - m) over this cache's tokens (m = -inf, l = 0, o = 0 for kv_len 0). */
LLAISYS_API int llaisysPagedAttentionDecodePartial(llaisysPagedKV_t kv, size_t layer, float *part, const void *q,
                                                   const int32_t *seq_ids, const int32_t *kv_lens, size_t n_seqs,
                                                   size_t nh, float scale);

/* One decode step from HOST buffers, synchronous -- the call a serving loop without device-resident activations makes.
 * Row i of k_new / v_new (host, [n_seqs, nkvh, head_dim]) becomes token kv_lens[i] - 1 of sequence seq_ids[i]; then
 * out[i] (host, [n_seqs, nh, head_dim]) = attention of q[i] (host) over the sequence's kv_lens[i] tokens. Pinned host
 * buffers make the copies asynchronous; pageable ones work. Buffers that are page-locked AND mapped into the device's
 * address space (cudaHostAlloc / cudaMallocHost, torch's pinned tensors) are read and written by the kernels directly
 * instead of through separate copies; they must not be touched until the call returns. Returns when out holds the
 * result. */
LLAISYS_API int llaisysPagedDecodeStepHost(llaisysPagedKV_t kv, size_t layer, void *out_host, const void *q_host,
                                           const void *k_new_host, const void *v_new_host, const int32_t *seq_ids,
                                           const int32_t *kv_lens, size_t n_seqs, size_t nh, float scale);

/* Log-sum-exp merge of n_parts partial results (each float [n_rows, head_dim + 2], packed back to back as
 * an all-gather leaves them) into out [n_rows, head_dim] of `dtype`, on the calling thread's current
 * runtime of `device_type`. */
LLAISYS_API int llaisysLseMerge(llaisysDeviceType_t device_type, int device_id, void *out, llaisysDataType_t dtype,
                                const float *parts, size_t n_parts, size_t n_rows, size_t head_dim);

/* ---- data path, device-resident index arrays, explicit stream --------------------------- */
/* No host validation, no staging copy, no synchronisation: safe to capture in a CUDA graph. The block
 * table must be current (llaisysPagedKVFlush). Out-of-range metadata is skipped and flagged
 * (llaisysPagedKVCheck). max_kv_len / max_q_len are upper bounds used to size the launch. */
LLAISYS_API int llaisysPagedKVAppendDev(llaisysPagedKV_t kv, size_t layer, const void *k_rows, const void *v_rows,
                                        const int32_t *seq_ids_dev, const int32_t *positions_dev, size_t n_rows,
                                        llaisysStream_t stream);
/* The step before attention, fused: qkv is the packed q|k|v projection [n_rows, (nh + 2 nkvh) * head_dim] of the cache's
 * dtype, bias an optional row of the same width (NULL = none). q and k heads get the half-split rotary embedding of the
 * reference's rope operator (angle = position / theta^(2j/d), computed in float; reference: README.md rope section,
 * test/ops/rope.py:11-32); rotated q is written to q_out [n_rows, nh, head_dim], rotated k and plain v go to token
 * positions_dev[i] of sequence seq_ids_dev[i]. One rounding to the dtype, after bias and rotation. */
LLAISYS_API int llaisysPagedKVRopeAppendDev(llaisysPagedKV_t kv, size_t layer, void *q_out, const void *qkv,
                                            const void *bias, const int32_t *seq_ids_dev, const int32_t *positions_dev,
                                            size_t n_rows, size_t nh, float theta, llaisysStream_t stream);
LLAISYS_API int llaisysPagedAttentionDecodeDev(llaisysPagedKV_t kv, size_t layer, void *out, const void *q,
                                               const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs,
                                               size_t max_kv_len, size_t nh, float scale, llaisysStream_t stream);
/* One decode step in ONE launch: row i of k_new / v_new ([n_seqs, nkvh, head_dim], device, 16-byte aligned) becomes
 * token kv_lens_dev[i] - 1 of sequence seq_ids_dev[i] -- the same bits llaisysPagedKVAppendDev would write -- and out[i]
 * is the attention of q[i] over the sequence's kv_lens_dev[i] tokens, the new one included. A sequence may appear once
 * per call. NVIDIA: pools of 16-bit data, head_dim 128, 16-token pages, nh / nkvh <= 8 (LLAISYS_E_UNSUPPORTED otherwise:
 * call AppendDev then DecodeDev). Takes part in launch overlap like the decode call. */
LLAISYS_API int llaisysPagedDecodeStepDev(llaisysPagedKV_t kv, size_t layer, void *out, const void *q, const void *k_new,
                                          const void *v_new, const int32_t *seq_ids_dev, const int32_t *kv_lens_dev,
                                          size_t n_seqs, size_t max_kv_len, size_t nh, float scale, llaisysStream_t stream);
LLAISYS_API int llaisysPagedAttentionDecodePartialDev(llaisysPagedKV_t kv, size_t layer, float *part, const void *q,
                                                      const int32_t *seq_ids_dev, const int32_t *kv_lens_dev,
                                                      size_t n_seqs, size_t max_kv_len, size_t nh, float scale,
                                                      llaisysStream_t stream);
/* q_starts_dev is int32 [n_seqs + 1]: row offset of each sequence's chunk in q / out. Attention calls on one cache
 * share its workspace (partial results of work that is split over CTAs) and must be ordered on one stream. */
LLAISYS_API int llaisysPagedAttentionPrefillDev(llaisysPagedKV_t kv, size_t layer, void *out, const void *q,
                                                const int32_t *seq_ids_dev, const int32_t *q_starts_dev,
                                                const int32_t *kv_lens_dev, size_t n_seqs, size_t total_q,
                                                size_t max_q_len, size_t max_kv_len, size_t nh, float scale,
                                                llaisysStream_t stream);

/* ---- decode without any allocation ------------------------------------------------------------- */
/* No counterpart in the reference. For callers that cannot let a library allocate device memory: a server that
 * has already given all free HBM to its own page pool (a library cudaMalloc would fail or fragment it), or a
 * decode loop that cannot afford the device-wide stall of an allocation or release. The caller passes its own
 * page pool of one layer (layout as above: [page][K|V][nkvh][16][128], BF16 or F16), its block table, the
 * per-sequence table rows (seq_ids_dev, or NULL for row i = sequence i) and lengths, q and out -- all device
 * memory -- and the split-KV scratch comes from a fixed array inside the library's device image instead of an
 * allocation.
 *   Limits: n_seqs * nkvh <= 512, nh / nkvh <= 8, head_dim 128, page size 16, GPUs of up to 160 SMs; larger
 *           requests return LLAISYS_E_INVALID and queue nothing. The array costs about 3.5 MiB on every GPU
 *           that loads the library, for the life of the process.
 *   Sharing: every call on a device uses the same array. What has to start at zero is cleared at the start of
 *           each call; calls that overlap on the GPU (unordered streams) race on it -- keep them ordered.
 *   First call on a device looks up the array's device address; make that call before any stream capture. A failed
 *           look-up is reported (LLAISYS_E_DEVICE) and tried again by the next call.
 *   Device: the call makes device_id current while it runs and restores the caller's current device before returning.
 * error_flag_dev (optional, device int32, caller-zeroed): receives the kErr bits if the kernel had to skip an
 * out-of-range page. NULL collects them in a word inside the library instead, which stays set until
 * llaisysPagedAttentionDecodeNoAllocStatus reads it -- a caller that passes NULL should poll that call. */
LLAISYS_API int llaisysPagedAttentionDecodeNoAlloc(int device_id, void *out, const void *q, void *pool_layer,
                                                   const int32_t *block_table_dev, size_t table_stride,
                                                   size_t num_pages, const int32_t *seq_ids_dev,
                                                   const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len,
                                                   size_t nh, size_t nkvh, llaisysDataType_t dtype, float scale,
                                                   int32_t *error_flag_dev, llaisysStream_t stream);
/* Synchronises `stream`, writes to *flags_out the error bits collected on device_id by no-alloc calls that passed no
 * error word of their own (0 = none; 1 = a page index was out of range and its page was skipped) and clears them.
 * Allocates nothing. No counterpart in the reference. */
LLAISYS_API int llaisysPagedAttentionDecodeNoAllocStatus(int device_id, llaisysStream_t stream, int32_t *flags_out);

/* ---- split-KV decode across the GPUs of one node through peer memory --------------------------------------------- */
/* For ONE long sequence whose KV range is cut across ranks (one process per GPU): instead of an all-gather through a
 * collective library, every rank's decode kernel stores the values of its partial (o, m, l) rows straight into slots of
 * all the ranks' exchange buffers over NVLink (buffers mapped with CUDA IPC; plain stores, nothing reads remote memory).
 * Every value travels as one 8-byte word together with the number of the step it belongs to, so a merge kernel can take
 * each value the moment it is current: no flag, no fence, two launches per step. Everything is queued on the given
 * stream and can be captured in a CUDA graph (the step counter lives on the device). Waits for peers are bounded: a
 * wait that runs out flags an error (llaisysPeerExchangeStatus) instead of hanging. */
typedef struct LlaisysPeerExchange *llaisysPeerExchange_t;

/* slot_floats: capacity for one rank's partial = rows * (head_dim + 2) floats, a multiple of 4. world <= 16. The
 * calling thread's current device (llaisysSetContextRuntime) must be the rank's GPU. */
LLAISYS_API int llaisysPeerExchangeCreate(llaisysPeerExchange_t *ex_out, int device_id, int rank, int world,
                                          size_t slot_floats);
LLAISYS_API void llaisysPeerExchangeDestroy(llaisysPeerExchange_t ex);
/* 64 bytes that let the other ranks map this rank's buffer; send them over any host channel. */
LLAISYS_API int llaisysPeerExchangeHandle(llaisysPeerExchange_t ex, void *out_64_bytes);
/* handles: world * 64 bytes, entry i from rank i. Every rank must call it once before the first step. */
LLAISYS_API int llaisysPeerExchangeConnect(llaisysPeerExchange_t ex, const void *handles);
/* Unmaps the other ranks' buffers (synchronises the device first). Shutting down: every rank disconnects, the ranks
 * meet on the host, then every rank destroys -- a buffer is released only when nobody maps it any more. */
LLAISYS_API int llaisysPeerExchangeDisconnect(llaisysPeerExchange_t ex);
/* Partial decode of this rank's slice (as llaisysPagedAttentionDecodePartialDev) + exchange + merge into out
 * [n_seqs, nh, head_dim]. Every rank passes the same q and its LOCAL sequences / lengths. */
LLAISYS_API int llaisysPagedAttentionDecodeSplitDev(llaisysPagedKV_t kv, size_t layer, void *out, const void *q,
                                                    const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs,
                                                    size_t max_kv_len, size_t nh, float scale, llaisysPeerExchange_t ex,
                                                    llaisysStream_t stream);
/* Polls (about half a microsecond each) after which the merge's wait for a peer's values gives up; the default is
 * about a second (2 << 20). Set it before the first step. After a wait has run out the step's output is undefined and the ranks' step
 * counters have diverged: every rank destroys its exchange and creates a new one before the next step. */
LLAISYS_API int llaisysPeerExchangeSetWaitLimit(llaisysPeerExchange_t ex, uint32_t polls);
/* Synchronises the stream; 0, or 1 when a wait for a peer ran out since the last call (cleared by the call). */
LLAISYS_API int llaisysPeerExchangeStatus(llaisysPeerExchange_t ex, llaisysStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* LLAISYS_PAGED_KV_H */
