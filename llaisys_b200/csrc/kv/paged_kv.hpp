// Paged KV cache: a fixed pool of pages, a free list, per-sequence block tables, and the data-path calls that
// read and write pages through them. New code -- the reference names a KV cache only as future work
// (README.md:316, :412, :424).
//
// Host state (block manager) is plain C++ and identical for CPU and NVIDIA caches; the device copy of the
// block table is refreshed lazily (only rows that changed) when a data-path call needs it.
#pragma once

#include "../kernels/args.hpp"
#include "../tensor/tensor.hpp"

#include <list>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace llaisys::kv {

// Thrown inside the library for every failure of the status-returning API; the C thunks turn it into a code.
struct StatusError : std::runtime_error {
    int code;
    StatusError(int code_, const std::string &what) : std::runtime_error(what), code(code_) {}
};

struct PagedKVConfig {
    llaisysDeviceType_t device_type = LLAISYS_DEVICE_CPU;
    int device_id = 0;
    llaisysDataType_t dtype = LLAISYS_DTYPE_BF16;
    size_t nlayer = 1, num_pages = 0, page_size = 16, nkvh = 0, head_dim = 0;
    size_t max_seqs = 0, max_pages_per_seq = 0;
};

class PagedKV {
public:
    explicit PagedKV(const PagedKVConfig &cfg);
    ~PagedKV() = default;
    PagedKV(const PagedKV &) = delete;
    PagedKV &operator=(const PagedKV &) = delete;

    const PagedKVConfig &config() const { return _cfg; }

    // ---- block manager (host only) ----
    int32_t seqAdd();
    void seqReserve(int32_t seq, size_t n_tokens);
    void seqAssignPages(int32_t seq, const int32_t *pages, size_t n_pages);
    void seqFree(int32_t seq);
    // Pages a reserve can still get: never-used or released pages plus cached ones (released, but still findable by
    // prefix; the least recently released is evicted first).
    size_t numFreePages() const { return _free_pages.size() + _lru.size(); }
    size_t numCachedPages() const { return _lru.size(); }
    int32_t pageRefCount(int32_t page) const;

    // ---- prefix sharing (host only, except the one-page copy of a fork) ----
    // New sequence that shares the parent's first n_tokens: whole pages by reference, a partial last page by copy (all
    // layers, queued on the calling thread's stream after everything already queued there).
    int32_t seqFork(int32_t parent, size_t n_tokens);
    // Registers the sequence's full pages under the chain of their token ids (tokens[0, n_tokens) are the ids of the
    // tokens whose K/V the sequence holds), so that later sequences starting with the same tokens can find them.
    // Incremental: pages hashed by an earlier call (or attached by a match) are not hashed again, so a caller may
    // publish after every step; the tokens of those pages must be the ones given before.
    void seqPublish(int32_t seq, const int64_t *tokens, size_t n_tokens);
    // Attaches to an EMPTY sequence the published pages matching the longest whole-page prefix of tokens[0, n_tokens);
    // -> number of tokens covered (a multiple of the page size).
    size_t seqMatchPrefix(int32_t seq, const int64_t *tokens, size_t n_tokens);
    size_t numSeqs() const { return _n_live; }
    int64_t seqNumPages(int32_t seq) const;
    void seqPages(int32_t seq, int32_t *pages_out, size_t cap) const;

    // ---- device-side views ----
    std::byte *poolData(size_t layer) const;
    size_t layerBytes() const { return _layer_bytes; }
    const int32_t *blockTableData() const { return reinterpret_cast<const int32_t *>(_table_dev->memory()); }
    void setLaunchOverlap(bool enable) { _overlap = enable; }
    // LLAISYS_KERNEL_* id of the kernel that served this cache's most recent attention call
    int lastKernel() const { return _last_kernel; }
    void flush(); // queue uploads of the table rows that changed since the last flush
    void check(); // synchronise, throw LLAISYS_E_KERNEL if a kernel flagged bad metadata

    // ---- data path: host index arrays (validated, staged, queued on the calling thread's stream) ----
    void append(size_t layer, const void *k_rows, const void *v_rows, const int32_t *seq_ids, const int32_t *positions,
                size_t n_rows);
    void gather(size_t layer, int32_t seq, size_t n_tokens, void *k_out, void *v_out);
    void decode(size_t layer, void *out, float *part, const void *q, const int32_t *seq_ids, const int32_t *kv_lens,
                size_t n_seqs, size_t nh, float scale);
    void prefill(size_t layer, void *out, const void *q, const int32_t *seq_ids, const int32_t *q_lens,
                 const int32_t *kv_lens, size_t n_seqs, size_t nh, float scale);
    // One decode step from HOST buffers, synchronous: row i of k_new / v_new [n_seqs, nkvh, d] becomes token
    // kv_lens[i] - 1 of sequence seq_ids[i], then out[i] = attention of q[i] over its kv_lens[i] tokens. On a device
    // cache: copies in, both kernels, copy out and one synchronise, all queued by this one call.
    void decodeStepHost(size_t layer, void *out_host, const void *q_host, const void *k_new_host, const void *v_new_host,
                        const int32_t *seq_ids, const int32_t *kv_lens, size_t n_seqs, size_t nh, float scale);

    // ---- data path: device index arrays, explicit stream (no validation, no staging) ----
    void appendDev(size_t layer, const void *k_rows, const void *v_rows, const int32_t *seq_ids_dev,
                   const int32_t *positions_dev, size_t n_rows, llaisysStream_t stream);
    // qkv [n_rows, (nh + 2 nkvh) * d] (+ optional bias row) -> rotated q in q_out [n_rows, nh, d], rotated k and v appended
    void ropeAppendDev(size_t layer, void *q_out, const void *qkv, const void *bias, const int32_t *seq_ids_dev,
                       const int32_t *positions_dev, size_t n_rows, size_t nh, float theta, llaisysStream_t stream);
    void decodeDev(size_t layer, void *out, float *part, const void *q, const int32_t *seq_ids_dev,
                   const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len, size_t nh, float scale,
                   llaisysStream_t stream);
    // One decode step in one launch: row i of k_new / v_new becomes token kv_lens[i] - 1 of sequence i, then attention of
    // q[i] over the kv_lens[i] tokens. Device caches: 16-bit, head_dim 128, page 16 pools only (the TMA decode kernel).
    void decodeStepDev(size_t layer, void *out, const void *q, const void *k_new, const void *v_new,
                       const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len, size_t nh,
                       float scale, llaisysStream_t stream);
    // Partial decode of this cache's slice of a KV-range split, its rows stored by the decode kernel itself into slot
    // `rank` of every rank's exchange buffer and this rank's flag stamped there when the last row is out. TMA pools only.
    bool canPushPartials(size_t nh) const { return onDevice() && fastShape() && nh % _cfg.nkvh == 0 && nh / _cfg.nkvh <= 8; }
    void decodeSplitDev(size_t layer, const void *q, const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs,
                        size_t max_kv_len, size_t nh, float scale, const kernels::PeerSink &peers, llaisysStream_t stream);
    void prefillDev(size_t layer, void *out, const void *q, const int32_t *seq_ids_dev, const int32_t *q_starts_dev,
                    const int32_t *kv_lens_dev, size_t n_seqs, size_t total_q, size_t max_q_len, size_t max_kv_len,
                    size_t nh, float scale, llaisysStream_t stream);

private:
    struct Seq {
        bool live = false;
        int32_t n_pages = 0;
        int32_t dirty_lo = 0, dirty_hi = 0; // table entries [lo, hi) not yet on the device
        bool queued_dirty = false;
        // prefix chain: pages [0, n_chained) have been hashed, chain_key is the key of page n_chained - 1
        int32_t n_chained = 0;
        uint64_t chain_key = 0;
    };

    struct PrefixEntry {
        int32_t page;
        uint64_t parent; // key of the page before it in the chain (0 for the first)
        std::vector<int64_t> tokens; // the page's token ids, to tell a match from a hash collision
    };

    int32_t takePage();           // from the free stack, else evict the oldest cached page
    void releasePage(int32_t page); // one reference less; at zero the page becomes cached (if published) or free
    void unpublish(int32_t page);
    uint64_t chainKey(uint64_t parent, const int64_t *tokens) const;
    Seq &liveSeq(int32_t seq);
    const Seq &liveSeq(int32_t seq) const;
    void markDirty(int32_t seq, int32_t lo, int32_t hi);
    void checkLayer(size_t layer) const;
    kernels::KVView view(size_t layer) const;
    core::Runtime &enter() const;                   // make the cache's device current on this thread
    int32_t *stage(const int32_t *const *arrays, const size_t *lens, size_t n_arrays); // host arrays -> device
    kernels::AttnScratch scratch() const;
    // 16-bit, head_dim 128, 16-token pages on a device: the shapes the TMA decode and tcgen05 chunk kernels serve
    bool fastShape() const { return _has_tma; }
    void launchDecode(size_t layer, void *out, float *part, const void *q, const void *k_new, const void *v_new,
                      const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len, size_t nh,
                      float scale, llaisysStream_t stream, bool overlap, const kernels::PeerSink *peers = nullptr,
                      const int32_t *host_seq_ids = nullptr, const int32_t *host_kv_lens = nullptr);
    bool onDevice() const { return _cfg.device_type != LLAISYS_DEVICE_CPU; }

    PagedKVConfig _cfg;
    size_t _elem = 0, _page_elems = 0, _layer_bytes = 0;

    // block manager
    std::vector<int32_t> _free_pages; // stack; back() is handed out next
    std::vector<int32_t> _page_ref;   // sequences holding the page; 0 = free or cached
    std::vector<uint64_t> _page_key;  // prefix-chain key the page is published under, 0 = not published
    std::list<int32_t> _lru;          // cached pages (ref 0, published), least recently released first
    std::vector<std::list<int32_t>::iterator> _lru_pos;
    std::unordered_map<uint64_t, PrefixEntry> _prefix_index;
    std::vector<Seq> _seqs;
    std::vector<int32_t> _free_seq_ids;
    std::vector<int32_t> _table_host; // [max_seqs][max_pages_per_seq]
    std::vector<int32_t> _dirty_seqs;
    size_t _n_live = 0;

    // device memory (host memory for a CPU cache)
    // _partials / _counters: split-KV and split-tile workspace of the attention kernels, sized for the largest call the
    // cache can take and allocated ONCE, at construction: captured graphs keep pointing at it, and no data-path call with
    // device index arrays ever allocates
    core::storage_t _pool, _table_dev, _error_dev, _meta_dev, _partials, _counters, _step_dev, _host_stage;
    size_t _step_cap = 0;
    size_t _meta_cap = 0, _partials_floats = 0, _counters_len = 0;
    std::vector<int32_t> _stage_buf, _step_positions;
    std::vector<uint32_t> _seen_mark; // per sequence: the step that last named it (duplicate check of the host step)
    uint32_t _seen_epoch = 0;
    const void *_host_stage_alias = nullptr; // device-side address of _host_stage (mapped page-locked memory)

    // TMA view of the pool (NVIDIA, 16-bit, head_dim 128, page 16 only); _has_tma is false otherwise
    alignas(64) unsigned char _tma_desc[128] = {};      // decode: box = K and V of a page
    alignas(64) unsigned char _tma_tile_desc[256] = {}; // prefill, two maps: box = one half-tile (K); box = one tile as two halves (V)
    bool _has_tma = false, _has_tma_tile = false;
    bool _overlap = false; // launch append / decode with programmatic stream serialisation
    int _last_kernel = 0;
};

// Picks the kernel for a batch on an NVIDIA device and queues it: split-KV decode or tensor-core prefill where
// the shape allows, the generic kernel otherwise. `scratch` may be empty when the shape cannot use it.
// -> the LLAISYS_KERNEL_* id of the kernel queued. Inside the specialised kernels' domain (16-bit, head_dim 128, page 16,
// group <= 8) a call the kernel cannot take throws LLAISYS_E_UNSUPPORTED with the reason; it is never re-routed.
int run_attention_nvidia(llaisysStream_t stream, llaisysDataType_t dtype, const kernels::KVView &view,
                         const kernels::AttnBatch &batch, const void *q, float scale, const kernels::AttnOut &out,
                         const kernels::AttnScratch &scratch);
// Kernel id of the calling thread's most recent attention call (any cache, or the legacy operator).
int lastAttentionKernel();
void noteAttentionKernel(int id);

} // namespace llaisys::kv
