#include "paged_kv.hpp"

#include "../common/check.hpp"
#include "../common/dtypes.hpp"
#include "../cpu/cpu_kernels.hpp"
#include "llaisys/paged_kv.h"
#ifdef ENABLE_NVIDIA_API
#include "../kernels/kernels.hpp"
#endif

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <sstream>

namespace llaisys::kv {

namespace {

template <typename... Args>
[[noreturn]] void fail(int code, Args &&...args) {
    std::ostringstream os;
    (os << ... << args);
    throw StatusError(code, os.str());
}

#define KV_REQUIRE(cond, code, ...) \
    do {                            \
        if (!(cond)) {              \
            fail(code, __VA_ARGS__); \
        }                           \
    } while (0)

constexpr size_t kMaxInt32 = size_t(std::numeric_limits<int32_t>::max());
constexpr size_t kMaxDecodeSeqs = 1024; // sequences per launch of the TMA decode kernel

} // namespace

// ---- construction ---------------------------------------------------------------------------------

PagedKV::PagedKV(const PagedKVConfig &cfg) : _cfg(cfg) {
    KV_REQUIRE(cfg.dtype == LLAISYS_DTYPE_F32 || cfg.dtype == LLAISYS_DTYPE_F16 || cfg.dtype == LLAISYS_DTYPE_BF16,
               LLAISYS_E_INVALID, "paged KV: dtype must be F32, F16 or BF16");
    KV_REQUIRE(cfg.nlayer > 0 && cfg.num_pages > 0 && cfg.page_size > 0 && cfg.nkvh > 0 && cfg.head_dim > 0 &&
                   cfg.max_seqs > 0 && cfg.max_pages_per_seq > 0,
               LLAISYS_E_INVALID, "paged KV: every size must be positive");
    KV_REQUIRE(cfg.num_pages <= kMaxInt32 && cfg.max_seqs <= kMaxInt32 && cfg.max_pages_per_seq <= kMaxInt32 &&
                   cfg.page_size * cfg.max_pages_per_seq <= kMaxInt32,
               LLAISYS_E_INVALID, "paged KV: sizes must fit 32-bit indices");
    _elem = utils::dsize(cfg.dtype);
    KV_REQUIRE((cfg.head_dim * _elem) % 16 == 0, LLAISYS_E_INVALID,
               "paged KV: a head row (head_dim * element size) must be a multiple of 16 bytes");
    _page_elems = 2 * cfg.nkvh * cfg.page_size * cfg.head_dim;
    _layer_bytes = cfg.num_pages * _page_elems * _elem;

    auto &ctx = core::context();
    KV_REQUIRE(cfg.device_type == LLAISYS_DEVICE_CPU || cfg.device_type == LLAISYS_DEVICE_NVIDIA, LLAISYS_E_INVALID,
               "paged KV: unknown device type");
    const int n_dev = llaisysGetRuntimeAPI(cfg.device_type)->get_device_count();
    KV_REQUIRE(cfg.device_id >= 0 && cfg.device_id < n_dev, LLAISYS_E_DEVICE, "paged KV: device ", cfg.device_id,
               " does not exist (", n_dev, " device(s) of this type)");
    ctx.setDevice(cfg.device_type, cfg.device_id);
    auto &rt = ctx.runtime();

    _pool = rt.allocateDeviceStorage(cfg.nlayer * _layer_bytes);
    _table_dev = rt.allocateDeviceStorage(cfg.max_seqs * cfg.max_pages_per_seq * sizeof(int32_t));
    _error_dev = rt.allocateDeviceStorage(sizeof(int32_t));
    // Pages start zeroed: tokens past a sequence's length are never read as data, but a tile load may touch
    // them, and zero keeps such lanes finite.
    if (onDevice()) {
#ifdef ENABLE_NVIDIA_API
        kernels::fill_zero(rt.stream(), _pool->memory(), _pool->size());
        kernels::fill_zero(rt.stream(), _table_dev->memory(), _table_dev->size());
        kernels::fill_zero(rt.stream(), _error_dev->memory(), _error_dev->size());
        rt.synchronize();
        if (_elem == 2 && cfg.head_dim == 128 && cfg.page_size == 16) {
            // one row of 128 elements per (layer, page, K|V, kv-head, slot)
            const uint64_t rows = uint64_t(cfg.nlayer) * cfg.num_pages * 2 * cfg.nkvh * cfg.page_size;
            _has_tma = kernels::make_kv_tensor_map(_tma_desc, _pool->memory(), rows, uint32_t(cfg.nkvh), cfg.dtype) == 0;
            _has_tma_tile =
                kernels::make_kv_tile_tensor_map(_tma_tile_desc, _pool->memory(), rows, uint32_t(cfg.nkvh), cfg.dtype) == 0;
            // These pools are served by the TMA decode kernel and the tcgen05 chunk kernel and by nothing else: a pool
            // they cannot address is refused here, not quietly handed to a slower kernel later.
            KV_REQUIRE(_has_tma && _has_tma_tile, LLAISYS_E_DEVICE,
                       "paged KV: no TMA tensor map for this pool (cuTensorMapEncodeTiled unavailable, or more than 2^31 "
                       "rows of 128 elements)");
            // Workspace of both kernels, for the largest call this cache can take (a decode call is cut into launches
            // of at most kMaxDecodeSeqs sequences; the chunk kernel's need does not depend on the batch).
            size_t floats = 0, counters = 0, f2 = 0, c2 = 0;
            const size_t seqs = std::min(cfg.max_seqs, kMaxDecodeSeqs);
            kernels::attention_decode_split_scratch(int32_t(seqs), int32_t(8 * cfg.nkvh), int32_t(cfg.nkvh), 128,
                                                    int32_t(cfg.page_size * cfg.max_pages_per_seq), &floats, &counters);
            kernels::attention_prefill_tc_scratch(&f2, &c2);
            _partials_floats = std::max(floats, f2);
            _counters_len = std::max(counters, c2);
            _partials = rt.allocateDeviceStorage(_partials_floats * sizeof(float));
            _counters = rt.allocateDeviceStorage(_counters_len * sizeof(int32_t));
            kernels::fill_zero(rt.stream(), _counters->memory(), _counters->size());
            rt.synchronize();
        }
        // index arrays of the host-buffer step are written here and read by a kernel: page-locked, mapped memory
        _host_stage = rt.allocateHostStorage((3 * cfg.max_seqs * sizeof(int32_t) + 15) / 16 * 16);
#endif
    } else {
        std::memset(_pool->memory(), 0, _pool->size());
        std::memset(_table_dev->memory(), 0, _table_dev->size());
        std::memset(_error_dev->memory(), 0, _error_dev->size());
    }

    _page_ref.assign(cfg.num_pages, 0);
    _page_key.assign(cfg.num_pages, 0);
    _lru_pos.assign(cfg.num_pages, _lru.end());
    _free_pages.resize(cfg.num_pages);
    for (size_t i = 0; i < cfg.num_pages; ++i) {
        _free_pages[i] = int32_t(cfg.num_pages - 1 - i); // page 0 is handed out first
    }
    _seqs.resize(cfg.max_seqs);
    _free_seq_ids.resize(cfg.max_seqs);
    for (size_t i = 0; i < cfg.max_seqs; ++i) {
        _free_seq_ids[i] = int32_t(cfg.max_seqs - 1 - i);
    }
    _table_host.assign(cfg.max_seqs * cfg.max_pages_per_seq, 0);
}

// ---- block manager ----------------------------------------------------------------------------------

PagedKV::Seq &PagedKV::liveSeq(int32_t seq) {
    KV_REQUIRE(seq >= 0 && size_t(seq) < _seqs.size() && _seqs[seq].live, LLAISYS_E_NO_SEQ, "paged KV: sequence ",
               seq, " does not exist");
    return _seqs[seq];
}
const PagedKV::Seq &PagedKV::liveSeq(int32_t seq) const { return const_cast<PagedKV *>(this)->liveSeq(seq); }

void PagedKV::markDirty(int32_t seq, int32_t lo, int32_t hi) {
    Seq &s = _seqs[seq];
    if (!s.queued_dirty) {
        s.queued_dirty = true;
        s.dirty_lo = lo;
        s.dirty_hi = hi;
        _dirty_seqs.push_back(seq);
    } else {
        s.dirty_lo = std::min(s.dirty_lo, lo);
        s.dirty_hi = std::max(s.dirty_hi, hi);
    }
}

int32_t PagedKV::seqAdd() {
    KV_REQUIRE(!_free_seq_ids.empty(), LLAISYS_E_NO_SEQ, "paged KV: all ", _cfg.max_seqs, " sequence slots are in use");
    const int32_t id = _free_seq_ids.back();
    _free_seq_ids.pop_back();
    Seq &s = _seqs[id];
    s.live = true;
    s.n_pages = 0;
    s.n_chained = 0;
    s.chain_key = 0;
    ++_n_live;
    return id;
}

void PagedKV::seqReserve(int32_t seq, size_t n_tokens) {
    Seq &s = liveSeq(seq);
    const size_t want_pages = (n_tokens + _cfg.page_size - 1) / _cfg.page_size;
    if (want_pages <= size_t(s.n_pages)) {
        return;
    }
    KV_REQUIRE(want_pages <= _cfg.max_pages_per_seq, LLAISYS_E_INVALID, "paged KV: ", n_tokens,
               " tokens need more than max_pages_per_seq = ", _cfg.max_pages_per_seq, " pages");
    const size_t extra = want_pages - size_t(s.n_pages);
    KV_REQUIRE(extra <= numFreePages(), LLAISYS_E_NO_PAGES, "paged KV: need ", extra, " more pages, ", numFreePages(),
               " free");
    int32_t *row = _table_host.data() + size_t(seq) * _cfg.max_pages_per_seq;
    const int32_t first = s.n_pages;
    for (size_t i = 0; i < extra; ++i) {
        const int32_t page = takePage();
        _page_ref[page] = 1;
        row[s.n_pages++] = page;
    }
    markDirty(seq, first, s.n_pages);
}

void PagedKV::seqAssignPages(int32_t seq, const int32_t *pages, size_t n_pages) {
    Seq &s = liveSeq(seq);
    if (n_pages == 0) {
        return;
    }
    KV_REQUIRE(pages != nullptr, LLAISYS_E_INVALID, "paged KV: pages is null");
    KV_REQUIRE(size_t(s.n_pages) + n_pages <= _cfg.max_pages_per_seq, LLAISYS_E_INVALID,
               "paged KV: sequence would exceed max_pages_per_seq = ", _cfg.max_pages_per_seq);
    // Validate everything before changing anything (all-or-nothing). A provisional reference mark catches a page
    // named twice in the same request; marks are rolled back if a later entry fails.
    for (size_t i = 0; i < n_pages; ++i) {
        const int32_t p = pages[i];
        const bool in_range = p >= 0 && size_t(p) < _cfg.num_pages;
        if (!in_range || _page_ref[p] != 0) {
            for (size_t k = 0; k < i; ++k) {
                _page_ref[pages[k]] = 0;
            }
            KV_REQUIRE(in_range, LLAISYS_E_INVALID, "paged KV: page ", p, " is out of range");
            fail(LLAISYS_E_NO_PAGES, "paged KV: page ", p, " is not free");
        }
        _page_ref[p] = -1;
    }
    for (size_t i = 0; i < n_pages; ++i) {
        unpublish(pages[i]); // a cached page named explicitly stops being findable: its contents are about to change
        _page_ref[pages[i]] = 1;
    }
    // remove the claimed pages from the free stack in one pass
    _free_pages.erase(std::remove_if(_free_pages.begin(), _free_pages.end(), [&](int32_t p) { return _page_ref[p] != 0; }),
                      _free_pages.end());
    int32_t *row = _table_host.data() + size_t(seq) * _cfg.max_pages_per_seq;
    const int32_t first = s.n_pages;
    for (size_t i = 0; i < n_pages; ++i) {
        row[s.n_pages++] = pages[i];
    }
    markDirty(seq, first, s.n_pages);
}

void PagedKV::seqFree(int32_t seq) {
    Seq &s = liveSeq(seq);
    const int32_t *row = _table_host.data() + size_t(seq) * _cfg.max_pages_per_seq;
    for (int32_t i = s.n_pages; i-- > 0;) { // reverse, so a re-reserve pops them in the original order
        releasePage(row[i]);
    }
    s.live = false;
    s.n_pages = 0;
    --_n_live;
    _free_seq_ids.push_back(seq);
}

// ---- page life cycle and prefix sharing ---------------------------------------------------------------------------

int32_t PagedKV::pageRefCount(int32_t page) const {
    if (page < 0 || size_t(page) >= _cfg.num_pages) {
        return -1;
    }
    return _page_ref[page];
}

void PagedKV::unpublish(int32_t page) {
    if (_page_key[page] != 0) {
        _prefix_index.erase(_page_key[page]);
        _page_key[page] = 0;
    }
    if (_lru_pos[page] != _lru.end()) {
        _lru.erase(_lru_pos[page]);
        _lru_pos[page] = _lru.end();
        if (_page_ref[page] == 0) {
            _free_pages.push_back(page);
        }
    }
}

int32_t PagedKV::takePage() {
    if (!_free_pages.empty()) {
        const int32_t page = _free_pages.back();
        _free_pages.pop_back();
        return page;
    }
    KV_REQUIRE(!_lru.empty(), LLAISYS_E_NO_PAGES, "paged KV: no free page");
    const int32_t page = _lru.front(); // the cached page released longest ago
    unpublish(page);                   // moves it to the free stack
    _free_pages.pop_back();
    return page;
}

void PagedKV::releasePage(int32_t page) {
    if (--_page_ref[page] > 0) {
        return;
    }
    if (_page_key[page] != 0) {
        _lru.push_back(page);
        _lru_pos[page] = std::prev(_lru.end());
    } else {
        _free_pages.push_back(page);
    }
}

// 64-bit chain key: the parent's key and the page's token ids through a multiply-xorshift mix; never 0.
uint64_t PagedKV::chainKey(uint64_t parent, const int64_t *tokens) const {
    uint64_t h = parent ^ 0x9e3779b97f4a7c15ull;
    for (size_t i = 0; i < _cfg.page_size; ++i) {
        h ^= uint64_t(tokens[i]) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        h *= 0xff51afd7ed558ccdull;
        h ^= h >> 33;
    }
    return h == 0 ? 1 : h;
}

void PagedKV::seqPublish(int32_t seq, const int64_t *tokens, size_t n_tokens) {
    Seq &s = liveSeq(seq);
    KV_REQUIRE(n_tokens <= size_t(s.n_pages) * _cfg.page_size, LLAISYS_E_INVALID, "paged KV publish: ", n_tokens,
               " tokens exceed the sequence's pages");
    const size_t full = n_tokens / _cfg.page_size;
    if (full <= size_t(s.n_chained)) {
        return;
    }
    KV_REQUIRE(tokens != nullptr, LLAISYS_E_INVALID, "paged KV publish: tokens is null");
    const int32_t *row = _table_host.data() + size_t(seq) * _cfg.max_pages_per_seq;
    uint64_t parent = s.chain_key;
    for (size_t i = size_t(s.n_chained); i < full; ++i) {
        const int64_t *chunk = tokens + i * _cfg.page_size;
        const uint64_t key = chainKey(parent, chunk);
        const int32_t page = row[i];
        if (_page_key[page] == 0 && _prefix_index.find(key) == _prefix_index.end()) {
            _prefix_index.emplace(key, PrefixEntry{page, parent, std::vector<int64_t>(chunk, chunk + _cfg.page_size)});
            _page_key[page] = key;
        }
        // else: this page is already published, or another page already holds the same prefix -- nothing to add
        parent = key;
    }
    s.n_chained = int32_t(full);
    s.chain_key = parent;
}

size_t PagedKV::seqMatchPrefix(int32_t seq, const int64_t *tokens, size_t n_tokens) {
    Seq &s = liveSeq(seq);
    KV_REQUIRE(s.n_pages == 0, LLAISYS_E_INVALID, "paged KV match: the sequence already owns pages");
    size_t full = n_tokens / _cfg.page_size;
    full = std::min(full, _cfg.max_pages_per_seq);
    if (full == 0) {
        return 0;
    }
    KV_REQUIRE(tokens != nullptr, LLAISYS_E_INVALID, "paged KV match: tokens is null");
    int32_t *row = _table_host.data() + size_t(seq) * _cfg.max_pages_per_seq;
    uint64_t parent = 0;
    for (size_t i = 0; i < full; ++i) {
        const int64_t *chunk = tokens + i * _cfg.page_size;
        const uint64_t key = chainKey(parent, chunk);
        auto it = _prefix_index.find(key);
        if (it == _prefix_index.end() || it->second.parent != parent ||
            !std::equal(chunk, chunk + _cfg.page_size, it->second.tokens.begin())) {
            break;
        }
        const int32_t page = it->second.page;
        if (_page_ref[page]++ == 0) { // cached: back in use
            _lru.erase(_lru_pos[page]);
            _lru_pos[page] = _lru.end();
        }
        row[s.n_pages++] = page;
        parent = key;
    }
    if (s.n_pages > 0) {
        markDirty(seq, 0, s.n_pages);
    }
    s.n_chained = s.n_pages;
    s.chain_key = parent;
    return size_t(s.n_pages) * _cfg.page_size;
}

int32_t PagedKV::seqFork(int32_t parent, size_t n_tokens) {
    const Seq &ps = liveSeq(parent);
    KV_REQUIRE(n_tokens <= size_t(ps.n_pages) * _cfg.page_size, LLAISYS_E_INVALID, "paged KV fork: ", n_tokens,
               " tokens exceed the parent's pages");
    const size_t full = n_tokens / _cfg.page_size, rest = n_tokens % _cfg.page_size;
    KV_REQUIRE(rest == 0 || numFreePages() >= 1, LLAISYS_E_NO_PAGES, "paged KV fork: no page for the copy of the last page");
    const int32_t child = seqAdd();
    Seq &cs = _seqs[child];
    const int32_t *prow = _table_host.data() + size_t(parent) * _cfg.max_pages_per_seq;
    int32_t *crow = _table_host.data() + size_t(child) * _cfg.max_pages_per_seq;
    for (size_t i = 0; i < full; ++i) {
        ++_page_ref[prow[i]];
        crow[cs.n_pages++] = prow[i];
    }
    if (rest != 0) {
        const int32_t src = prow[full], dst = takePage();
        _page_ref[dst] = 1;
        crow[cs.n_pages++] = dst;
        const size_t page_bytes = _page_elems * _elem;
        auto &rt = enter();
        for (size_t l = 0; l < _cfg.nlayer; ++l) {
            std::byte *base = _pool->memory() + l * _layer_bytes;
            if (onDevice()) {
                rt.api()->memcpy_async(base + size_t(dst) * page_bytes, base + size_t(src) * page_bytes, page_bytes,
                                       LLAISYS_MEMCPY_D2D, rt.stream());
            } else {
                std::memcpy(base + size_t(dst) * page_bytes, base + size_t(src) * page_bytes, page_bytes);
            }
        }
    }
    if (cs.n_pages > 0) {
        markDirty(child, 0, cs.n_pages);
    }
    return child;
}

int64_t PagedKV::seqNumPages(int32_t seq) const {
    if (seq < 0 || size_t(seq) >= _seqs.size() || !_seqs[seq].live) {
        return -1;
    }
    return _seqs[seq].n_pages;
}

void PagedKV::seqPages(int32_t seq, int32_t *pages_out, size_t cap) const {
    const Seq &s = liveSeq(seq);
    const size_t n = std::min(cap, size_t(s.n_pages));
    if (n > 0) {
        KV_REQUIRE(pages_out != nullptr, LLAISYS_E_INVALID, "paged KV: pages_out is null");
        std::memcpy(pages_out, _table_host.data() + size_t(seq) * _cfg.max_pages_per_seq, n * sizeof(int32_t));
    }
}

// ---- device views -----------------------------------------------------------------------------------

void PagedKV::checkLayer(size_t layer) const {
    KV_REQUIRE(layer < _cfg.nlayer, LLAISYS_E_INVALID, "paged KV: layer ", layer, " out of range (", _cfg.nlayer, ")");
}

std::byte *PagedKV::poolData(size_t layer) const {
    checkLayer(layer);
    return _pool->memory() + layer * _layer_bytes;
}

kernels::KVView PagedKV::view(size_t layer) const {
    kernels::KVView v;
    v.k_base = poolData(layer);
    v.v_base = poolData(layer) + _cfg.nkvh * _cfg.page_size * _cfg.head_dim * _elem;
    v.page_stride = int64_t(_page_elems);
    v.head_stride = int64_t(_cfg.page_size * _cfg.head_dim);
    v.token_stride = int64_t(_cfg.head_dim);
    v.block_table = blockTableData();
    v.table_stride = int32_t(_cfg.max_pages_per_seq);
    v.page_size = int32_t(_cfg.page_size);
    v.num_pages = int32_t(_cfg.num_pages);
    v.nkvh = int32_t(_cfg.nkvh);
    v.d = int32_t(_cfg.head_dim);
    v.overlap_launch = _overlap;
    if (_has_tma_tile) {
        v.tma_tile_desc = _tma_tile_desc;
        v.tma_page0 = int64_t(layer) * int64_t(_cfg.num_pages);
    }
    if (_has_tma) {
        v.tma_desc = _tma_desc;
        v.tma_page0 = int64_t(layer) * int64_t(_cfg.num_pages);
    }
    return v;
}

core::Runtime &PagedKV::enter() const {
    auto &ctx = core::context();
    ctx.setDevice(_cfg.device_type, _cfg.device_id);
    return ctx.runtime();
}

void PagedKV::flush() {
    if (_dirty_seqs.empty()) {
        return;
    }
    auto &rt = enter();
    auto *dev = reinterpret_cast<int32_t *>(_table_dev->memory());
    for (int32_t seq : _dirty_seqs) {
        Seq &s = _seqs[seq];
        s.queued_dirty = false;
        if (!s.live || s.dirty_hi <= s.dirty_lo) {
            continue;
        }
        const size_t off = size_t(seq) * _cfg.max_pages_per_seq + size_t(s.dirty_lo);
        const size_t bytes = size_t(s.dirty_hi - s.dirty_lo) * sizeof(int32_t);
        // The source is ordinary pageable memory: the runtime stages it before the call returns, so the host
        // table may change again straight away.
        rt.api()->memcpy_async(dev + off, _table_host.data() + off, bytes, LLAISYS_MEMCPY_H2D, rt.stream());
    }
    _dirty_seqs.clear();
}

void PagedKV::check() {
    auto &rt = enter();
    rt.synchronize();
    int32_t word = 0;
    rt.api()->memcpy_sync(&word, _error_dev->memory(), sizeof(word), LLAISYS_MEMCPY_D2H);
    if (word != 0) {
        const int32_t zero = 0;
        rt.api()->memcpy_sync(_error_dev->memory(), &zero, sizeof(zero), LLAISYS_MEMCPY_H2D);
        fail(LLAISYS_E_KERNEL, "paged KV: a kernel skipped out-of-range metadata (flags 0x", std::hex, word,
             std::dec, ": 1 = page, 2 = position, 4 = sequence)");
    }
}

// Copies several small host arrays, back to back, into the cache's device-side metadata buffer and returns its
// base; array i starts at the sum of the lengths before it. One copy per call.
int32_t *PagedKV::stage(const int32_t *const *arrays, const size_t *lens, size_t n_arrays) {
    size_t total = 0;
    for (size_t i = 0; i < n_arrays; ++i) {
        total += lens[i];
    }
    auto &rt = enter();
    if (total > _meta_cap) {
        _meta_cap = std::max<size_t>(total * 2, 1024);
        _meta_dev = rt.allocateDeviceStorage(_meta_cap * sizeof(int32_t));
    }
    _stage_buf.resize(total);
    size_t at = 0;
    for (size_t i = 0; i < n_arrays; ++i) {
        std::memcpy(_stage_buf.data() + at, arrays[i], lens[i] * sizeof(int32_t));
        at += lens[i];
    }
    auto *dev = reinterpret_cast<int32_t *>(_meta_dev->memory());
    if (total > 0) {
        rt.api()->memcpy_async(dev, _stage_buf.data(), total * sizeof(int32_t), LLAISYS_MEMCPY_H2D, rt.stream());
    }
    return dev;
}

kernels::AttnScratch PagedKV::scratch() const {
    kernels::AttnScratch sc;
    sc.error_flag = reinterpret_cast<int32_t *>(_error_dev->memory());
    sc.partials = _partials ? reinterpret_cast<float *>(_partials->memory()) : nullptr;
    sc.partials_floats = _partials_floats;
    sc.counters = _counters ? reinterpret_cast<int32_t *>(_counters->memory()) : nullptr;
    sc.counters_len = _counters_len;
    return sc;
}

// ---- data path, device index arrays -----------------------------------------------------------------

void PagedKV::appendDev(size_t layer, const void *k_rows, const void *v_rows, const int32_t *seq_ids_dev,
                        const int32_t *positions_dev, size_t n_rows, llaisysStream_t stream) {
    checkLayer(layer);
    KV_REQUIRE(n_rows <= kMaxInt32, LLAISYS_E_INVALID, "paged KV: too many rows");
    if (n_rows == 0) {
        return;
    }
    KV_REQUIRE(k_rows && v_rows && seq_ids_dev && positions_dev, LLAISYS_E_INVALID, "paged KV append: null argument");
    const kernels::KVView v = view(layer);
    if (!onDevice()) {
        const int err = cpu::paged_append(_elem, v, k_rows, v_rows, seq_ids_dev, positions_dev, int32_t(n_rows),
                                          int32_t(_cfg.max_pages_per_seq));
        *reinterpret_cast<int32_t *>(_error_dev->memory()) |= err;
        return;
    }
#ifdef ENABLE_NVIDIA_API
    enter();
    kernels::paged_append(stream, _elem, v, k_rows, v_rows, seq_ids_dev, positions_dev, int32_t(n_rows),
                          int32_t(_cfg.max_pages_per_seq), reinterpret_cast<int32_t *>(_error_dev->memory()));
#else
    (void)stream;
    fail(LLAISYS_E_UNSUPPORTED, "this build has no NVIDIA backend");
#endif
}

void PagedKV::ropeAppendDev(size_t layer, void *q_out, const void *qkv, const void *bias, const int32_t *seq_ids_dev,
                            const int32_t *positions_dev, size_t n_rows, size_t nh, float theta, llaisysStream_t stream) {
    checkLayer(layer);
    KV_REQUIRE(n_rows <= kMaxInt32 && nh > 0 && nh <= 4096, LLAISYS_E_INVALID, "paged KV rope append: bad sizes");
    KV_REQUIRE(_cfg.head_dim % 2 == 0, LLAISYS_E_INVALID, "paged KV rope append: head_dim must be even");
    if (n_rows == 0) {
        return;
    }
    KV_REQUIRE(q_out && qkv && seq_ids_dev && positions_dev, LLAISYS_E_INVALID, "paged KV rope append: null argument");
    const kernels::KVView v = view(layer);
    if (!onDevice()) {
        const int err = cpu::paged_rope_append(_cfg.dtype, v, q_out, qkv, bias, seq_ids_dev, positions_dev, int32_t(n_rows),
                                               int32_t(nh), theta, int32_t(_cfg.max_pages_per_seq));
        *reinterpret_cast<int32_t *>(_error_dev->memory()) |= err;
        return;
    }
#ifdef ENABLE_NVIDIA_API
    enter();
    kernels::paged_rope_append(stream, _cfg.dtype, v, q_out, qkv, bias, seq_ids_dev, positions_dev, int32_t(n_rows),
                               int32_t(nh), theta, int32_t(_cfg.max_pages_per_seq),
                               reinterpret_cast<int32_t *>(_error_dev->memory()));
#else
    (void)stream;
    fail(LLAISYS_E_UNSUPPORTED, "this build has no NVIDIA backend");
#endif
}

void PagedKV::decodeDev(size_t layer, void *out, float *part, const void *q, const int32_t *seq_ids_dev,
                        const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len, size_t nh, float scale,
                        llaisysStream_t stream) {
    checkLayer(layer);
    KV_REQUIRE(nh > 0 && nh % _cfg.nkvh == 0, LLAISYS_E_INVALID, "paged attention: nh = ", nh,
               " is not a multiple of nkvh = ", _cfg.nkvh);
    KV_REQUIRE(n_seqs <= kMaxInt32 && max_kv_len <= _cfg.page_size * _cfg.max_pages_per_seq, LLAISYS_E_INVALID,
               "paged attention: batch or context too large for this cache");
    if (n_seqs == 0) {
        return;
    }
    KV_REQUIRE((out != nullptr) != (part != nullptr), LLAISYS_E_INVALID, "paged attention: exactly one output");
    KV_REQUIRE(q && seq_ids_dev && kv_lens_dev, LLAISYS_E_INVALID, "paged attention: null argument");
    launchDecode(layer, out, part, q, nullptr, nullptr, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh, scale, stream,
                 _overlap);
}

void PagedKV::decodeStepDev(size_t layer, void *out, const void *q, const void *k_new, const void *v_new,
                            const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len,
                            size_t nh, float scale, llaisysStream_t stream) {
    checkLayer(layer);
    KV_REQUIRE(nh > 0 && nh % _cfg.nkvh == 0, LLAISYS_E_INVALID, "paged decode step: nh = ", nh,
               " is not a multiple of nkvh = ", _cfg.nkvh);
    KV_REQUIRE(n_seqs <= kMaxInt32 && max_kv_len <= _cfg.page_size * _cfg.max_pages_per_seq, LLAISYS_E_INVALID,
               "paged decode step: batch or context too large for this cache");
    if (n_seqs == 0) {
        return;
    }
    KV_REQUIRE(out && q && k_new && v_new && seq_ids_dev && kv_lens_dev, LLAISYS_E_INVALID,
               "paged decode step: null argument");
    if (!onDevice()) {
        // host memory: the arrays can be read here
        std::vector<int32_t> pos(n_seqs);
        for (size_t i = 0; i < n_seqs; ++i) {
            pos[i] = kv_lens_dev[i] - 1;
        }
        appendDev(layer, k_new, v_new, seq_ids_dev, pos.data(), n_seqs, nullptr);
        decodeDev(layer, out, nullptr, q, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh, scale, nullptr);
        return;
    }
    KV_REQUIRE(fastShape() && nh / _cfg.nkvh <= 8, LLAISYS_E_UNSUPPORTED,
               "paged decode step: the one-launch step needs a 16-bit pool with head_dim 128, 16-token pages and at most 8 "
               "query heads per kv head; use llaisysPagedKVAppendDev + llaisysPagedAttentionDecodeDev");
    launchDecode(layer, out, nullptr, q, k_new, v_new, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh, scale, stream,
                 _overlap);
}

void PagedKV::decodeSplitDev(size_t layer, const void *q, const int32_t *seq_ids_dev, const int32_t *kv_lens_dev,
                             size_t n_seqs, size_t max_kv_len, size_t nh, float scale, const kernels::PeerSink &peers,
                             llaisysStream_t stream) {
    checkLayer(layer);
    KV_REQUIRE(nh > 0 && nh % _cfg.nkvh == 0, LLAISYS_E_INVALID, "split decode: nh = ", nh, " is not a multiple of nkvh = ",
               _cfg.nkvh);
    KV_REQUIRE(n_seqs >= 1 && n_seqs <= kMaxDecodeSeqs && max_kv_len <= _cfg.page_size * _cfg.max_pages_per_seq,
               LLAISYS_E_INVALID, "split decode: 1 to 1024 sequences per call, context within the cache's tables");
    KV_REQUIRE(q && seq_ids_dev && kv_lens_dev, LLAISYS_E_INVALID, "split decode: null argument");
    KV_REQUIRE(onDevice() && fastShape() && nh / _cfg.nkvh <= 8, LLAISYS_E_UNSUPPORTED,
               "split decode with the exchange in the kernel needs a 16-bit device pool, head_dim 128, 16-token pages");
    launchDecode(layer, nullptr, nullptr, q, nullptr, nullptr, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh, scale, stream,
                 _overlap, &peers);
}

// The decode kernel for one call, cut into launches of at most kMaxDecodeSeqs sequences (they share the workspace and
// run in stream order). k_new / v_new non-null: fused step.
void PagedKV::launchDecode(size_t layer, void *out, float *part, const void *q, const void *k_new, const void *v_new,
                           const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len,
                           size_t nh, float scale, llaisysStream_t stream, bool overlap, const kernels::PeerSink *peers,
                           const int32_t *host_seq_ids, const int32_t *host_kv_lens) {
    kernels::KVView v = view(layer);
    v.overlap_launch = overlap;
    const size_t d = _cfg.head_dim;
    for (size_t at = 0; at < n_seqs; at += kMaxDecodeSeqs) {
        kernels::AttnBatch b;
        b.seq_ids = seq_ids_dev ? seq_ids_dev + at : nullptr;
        b.kv_lens = kv_lens_dev ? kv_lens_dev + at : nullptr;
        b.host_seq_ids = host_seq_ids ? host_seq_ids + at : nullptr;
        b.host_kv_lens = host_kv_lens ? host_kv_lens + at : nullptr;
        b.const_q_len = 1;
        b.n_seqs = int32_t(std::min(kMaxDecodeSeqs, n_seqs - at));
        b.total_q = b.n_seqs;
        b.max_q_len = 1;
        b.max_kv_len = int32_t(max_kv_len);
        b.nh = int32_t(nh);
        kernels::AttnOut o;
        o.out = out ? static_cast<std::byte *>(out) + at * nh * d * _elem : nullptr;
        o.part = part ? part + at * nh * (d + 2) : nullptr;
        o.peers = peers;
        const std::byte *q_at = static_cast<const std::byte *>(q) + at * nh * d * _elem;
        if (!onDevice()) {
            const int err = cpu::attention(_cfg.dtype, v, b, q_at, scale, o);
            *reinterpret_cast<int32_t *>(_error_dev->memory()) |= err;
            _last_kernel = LLAISYS_KERNEL_CPU;
            noteAttentionKernel(_last_kernel);
            continue;
        }
#ifdef ENABLE_NVIDIA_API
        enter();
        if (k_new != nullptr) {
            const size_t row_bytes = _cfg.nkvh * d * _elem;
            const char *why = nullptr;
            if (kernels::attention_decode_tma(stream, _cfg.dtype, v, b, q_at, scale, o, scratch(),
                                              static_cast<const std::byte *>(k_new) + at * row_bytes,
                                              static_cast<const std::byte *>(v_new) + at * row_bytes, &why) != 0) {
                fail(LLAISYS_E_UNSUPPORTED, "paged decode step (TMA kernel): ", why ? why : "call not covered");
            }
            _last_kernel = LLAISYS_KERNEL_DECODE_TMA_FUSED;
            noteAttentionKernel(_last_kernel);
        } else {
            _last_kernel = run_attention_nvidia(stream, _cfg.dtype, v, b, q_at, scale, o, scratch());
        }
#else
        (void)stream;
        (void)k_new;
        (void)v_new;
        fail(LLAISYS_E_UNSUPPORTED, "this build has no NVIDIA backend");
#endif
    }
}

void PagedKV::prefillDev(size_t layer, void *out, const void *q, const int32_t *seq_ids_dev,
                         const int32_t *q_starts_dev, const int32_t *kv_lens_dev, size_t n_seqs, size_t total_q,
                         size_t max_q_len, size_t max_kv_len, size_t nh, float scale, llaisysStream_t stream) {
    checkLayer(layer);
    KV_REQUIRE(nh > 0 && nh % _cfg.nkvh == 0, LLAISYS_E_INVALID, "paged attention: nh = ", nh,
               " is not a multiple of nkvh = ", _cfg.nkvh);
    KV_REQUIRE(n_seqs <= kMaxInt32 && total_q <= kMaxInt32 && max_kv_len <= _cfg.page_size * _cfg.max_pages_per_seq,
               LLAISYS_E_INVALID, "paged attention: batch or context too large for this cache");
    if (n_seqs == 0 || total_q == 0) {
        return;
    }
    KV_REQUIRE(out && q && seq_ids_dev && q_starts_dev && kv_lens_dev, LLAISYS_E_INVALID,
               "paged attention: null argument");
    const kernels::KVView v = view(layer);
    kernels::AttnBatch b;
    b.seq_ids = seq_ids_dev;
    b.kv_lens = kv_lens_dev;
    b.q_starts = q_starts_dev;
    b.n_seqs = int32_t(n_seqs);
    b.total_q = int32_t(total_q);
    b.max_q_len = int32_t(max_q_len);
    b.max_kv_len = int32_t(max_kv_len);
    b.nh = int32_t(nh);
    kernels::AttnOut o;
    o.out = out;
    if (!onDevice()) {
        const int err = cpu::attention(_cfg.dtype, v, b, q, scale, o);
        *reinterpret_cast<int32_t *>(_error_dev->memory()) |= err;
        _last_kernel = LLAISYS_KERNEL_CPU;
        noteAttentionKernel(_last_kernel);
        return;
    }
#ifdef ENABLE_NVIDIA_API
    enter();
    _last_kernel = run_attention_nvidia(stream, _cfg.dtype, v, b, q, scale, o, scratch());
#else
    (void)stream;
    fail(LLAISYS_E_UNSUPPORTED, "this build has no NVIDIA backend");
#endif
}

// ---- data path, host index arrays -------------------------------------------------------------------

void PagedKV::append(size_t layer, const void *k_rows, const void *v_rows, const int32_t *seq_ids,
                     const int32_t *positions, size_t n_rows) {
    checkLayer(layer);
    if (n_rows == 0) {
        return;
    }
    KV_REQUIRE(k_rows && v_rows && seq_ids && positions, LLAISYS_E_INVALID, "paged KV append: null argument");
    for (size_t i = 0; i < n_rows; ++i) {
        const Seq &s = liveSeq(seq_ids[i]);
        KV_REQUIRE(positions[i] >= 0 && size_t(positions[i]) < size_t(s.n_pages) * _cfg.page_size, LLAISYS_E_INVALID,
                   "paged KV append: row ", i, " position ", positions[i], " is beyond the ", s.n_pages,
                   " page(s) reserved for sequence ", seq_ids[i]);
    }
    flush();
    if (!onDevice()) {
        return appendDev(layer, k_rows, v_rows, seq_ids, positions, n_rows, nullptr);
    }
    const int32_t *arrays[2] = {seq_ids, positions};
    const size_t lens[2] = {n_rows, n_rows};
    int32_t *dev = stage(arrays, lens, 2);
    appendDev(layer, k_rows, v_rows, dev, dev + n_rows, n_rows, enter().stream());
}

void PagedKV::gather(size_t layer, int32_t seq, size_t n_tokens, void *k_out, void *v_out) {
    checkLayer(layer);
    const Seq &s = liveSeq(seq);
    KV_REQUIRE(n_tokens <= size_t(s.n_pages) * _cfg.page_size, LLAISYS_E_INVALID, "paged KV gather: ", n_tokens,
               " tokens exceed the sequence's capacity");
    if (n_tokens == 0) {
        return;
    }
    KV_REQUIRE(k_out && v_out, LLAISYS_E_INVALID, "paged KV gather: null output");
    flush();
    const kernels::KVView v = view(layer);
    if (!onDevice()) {
        const int err = cpu::paged_gather(_elem, v, seq, int32_t(n_tokens), k_out, v_out);
        *reinterpret_cast<int32_t *>(_error_dev->memory()) |= err;
        return;
    }
#ifdef ENABLE_NVIDIA_API
    auto &rt = enter();
    kernels::paged_gather(rt.stream(), _elem, v, seq, int32_t(n_tokens), k_out, v_out,
                          reinterpret_cast<int32_t *>(_error_dev->memory()));
#else
    fail(LLAISYS_E_UNSUPPORTED, "this build has no NVIDIA backend");
#endif
}

void PagedKV::decode(size_t layer, void *out, float *part, const void *q, const int32_t *seq_ids,
                     const int32_t *kv_lens, size_t n_seqs, size_t nh, float scale) {
    checkLayer(layer);
    if (n_seqs == 0) {
        return;
    }
    KV_REQUIRE(seq_ids && kv_lens, LLAISYS_E_INVALID, "paged attention: null index array");
    size_t max_kv = 0;
    for (size_t i = 0; i < n_seqs; ++i) {
        const Seq &s = liveSeq(seq_ids[i]);
        KV_REQUIRE(kv_lens[i] >= 0 && size_t(kv_lens[i]) <= size_t(s.n_pages) * _cfg.page_size, LLAISYS_E_INVALID,
                   "paged attention: kv_len ", kv_lens[i], " exceeds the ", s.n_pages,
                   " page(s) reserved for sequence ", seq_ids[i]);
        max_kv = std::max(max_kv, size_t(kv_lens[i]));
    }
    flush();
    if (!onDevice()) {
        return decodeDev(layer, out, part, q, seq_ids, kv_lens, n_seqs, max_kv, nh, scale, nullptr);
    }
    const int32_t *arrays[2] = {seq_ids, kv_lens};
    const size_t lens[2] = {n_seqs, n_seqs};
    int32_t *dev = stage(arrays, lens, 2);
    decodeDev(layer, out, part, q, dev, dev + n_seqs, n_seqs, max_kv, nh, scale, enter().stream());
}

void PagedKV::decodeStepHost(size_t layer, void *out_host, const void *q_host, const void *k_new_host,
                             const void *v_new_host, const int32_t *seq_ids, const int32_t *kv_lens, size_t n_seqs,
                             size_t nh, float scale) {
    checkLayer(layer);
    if (n_seqs == 0) {
        return;
    }
    KV_REQUIRE(out_host && q_host && k_new_host && v_new_host && seq_ids && kv_lens, LLAISYS_E_INVALID,
               "paged decode step: null argument");
    KV_REQUIRE(nh > 0 && nh % _cfg.nkvh == 0, LLAISYS_E_INVALID, "paged attention: nh = ", nh,
               " is not a multiple of nkvh = ", _cfg.nkvh);
    KV_REQUIRE(n_seqs <= _cfg.max_seqs, LLAISYS_E_INVALID, "paged decode step: more rows than the cache has sequences");
    size_t max_kv = 0;
    std::vector<int32_t> &pos = _step_positions;
    pos.resize(n_seqs);
    _seen_mark.resize(_cfg.max_seqs, 0);
    if (++_seen_epoch == 0) { // wrapped: forget every mark
        std::fill(_seen_mark.begin(), _seen_mark.end(), 0u);
        _seen_epoch = 1;
    }
    for (size_t i = 0; i < n_seqs; ++i) {
        const Seq &s = liveSeq(seq_ids[i]);
        KV_REQUIRE(kv_lens[i] >= 1 && size_t(kv_lens[i]) <= size_t(s.n_pages) * _cfg.page_size, LLAISYS_E_INVALID,
                   "paged decode step: kv_len ", kv_lens[i], " is outside the ", s.n_pages,
                   " page(s) reserved for sequence ", seq_ids[i]);
        // two rows of one sequence would be written to the same slot by different warps
        KV_REQUIRE(_seen_mark[size_t(seq_ids[i])] != _seen_epoch, LLAISYS_E_INVALID, "paged decode step: sequence ",
                   seq_ids[i], " appears twice in one step");
        _seen_mark[size_t(seq_ids[i])] = _seen_epoch;
        pos[i] = kv_lens[i] - 1;
        max_kv = std::max(max_kv, size_t(kv_lens[i]));
    }
    flush();
    if (!onDevice()) {
        appendDev(layer, k_new_host, v_new_host, seq_ids, pos.data(), n_seqs, nullptr);
        decodeDev(layer, out_host, nullptr, q_host, seq_ids, kv_lens, n_seqs, max_kv, nh, scale, nullptr);
        return;
    }
    auto &rt = enter();
    const size_t q_bytes = n_seqs * nh * _cfg.head_dim * _elem, kv_bytes = n_seqs * _cfg.nkvh * _cfg.head_dim * _elem;
    const size_t need = 2 * q_bytes + 2 * kv_bytes; // q | out | k | v, each a multiple of 16 bytes
    if (need > _step_cap) {
        _step_cap = need * 2;
        _step_dev = rt.allocateDeviceStorage(_step_cap);
    }
    std::byte *q_d = _step_dev->memory(), *out_d = q_d + q_bytes, *k_d = out_d + q_bytes, *v_d = k_d + kv_bytes;
    const auto *api = rt.api();
    llaisysStream_t stream = rt.stream();
#ifdef ENABLE_NVIDIA_API
    if (fastShape() && nh / _cfg.nkvh <= 8) {
        // Two launches and no copy-engine transfer when the caller's buffers are page-locked and mapped (each small
        // copy costs more in set-up than in transfer): a copy kernel brings q to the device -- q is read by every CTA
        // that works on its sequence, so it is not left in host memory -- and the one-launch step reads each new K/V row
        // once, straight from the caller's memory, and stores each output row once, straight into it. Batches of up to
        // 256 sequences hand their index arrays to the step kernel by value, with the launch: nothing of them is
        // uploaded, and the kernel (launched to overlap the copy kernel) starts its page copies at once and waits for
        // q only where it needs it.
        const void *q_alias = kernels::mapped_host_alias(q_host, q_bytes);
        const void *k_alias = kernels::mapped_host_alias(k_new_host, kv_bytes);
        const void *v_alias = kernels::mapped_host_alias(v_new_host, kv_bytes);
        const void *out_alias = kernels::mapped_host_alias(out_host, q_bytes);
        auto aligned = [](const void *p) { return p != nullptr && reinterpret_cast<uintptr_t>(p) % 16 == 0; };
        const void *k_src = k_d, *v_src = v_d;
        if (aligned(k_alias) && aligned(v_alias)) {
            k_src = k_alias;
            v_src = v_alias;
        } else {
            api->memcpy_async(k_d, k_new_host, kv_bytes, LLAISYS_MEMCPY_H2D, stream);
            api->memcpy_async(v_d, v_new_host, kv_bytes, LLAISYS_MEMCPY_H2D, stream);
        }
        void *out_dst = aligned(out_alias) ? const_cast<void *>(out_alias) : out_d;
        const bool q_by_kernel = aligned(q_alias) && q_bytes % 16 == 0;
        if (n_seqs <= 256) {
            if (q_by_kernel) {
                const void *src[1] = {q_alias};
                void *dst[1] = {q_d};
                const size_t bytes[1] = {q_bytes};
                kernels::small_copies(stream, src, dst, bytes, 1);
            } else {
                api->memcpy_async(q_d, q_host, q_bytes, LLAISYS_MEMCPY_H2D, stream);
            }
            launchDecode(layer, out_dst, nullptr, q_d, k_src, v_src, nullptr, nullptr, n_seqs, max_kv, nh, scale, stream,
                         /*overlap=*/q_by_kernel, nullptr, seq_ids, kv_lens);
        } else {
            const size_t idx_bytes = (2 * n_seqs * sizeof(int32_t) + 15) / 16 * 16;
            if (idx_bytes / sizeof(int32_t) > _meta_cap) {
                _meta_cap = std::max<size_t>(idx_bytes / sizeof(int32_t) * 2, 1024);
                _meta_dev = rt.allocateDeviceStorage(_meta_cap * sizeof(int32_t));
            }
            auto *idx_host = reinterpret_cast<int32_t *>(_host_stage->memory()); // free: the previous step has synchronised
            std::memcpy(idx_host, seq_ids, n_seqs * sizeof(int32_t));
            std::memcpy(idx_host + n_seqs, kv_lens, n_seqs * sizeof(int32_t));
            auto *idx = reinterpret_cast<int32_t *>(_meta_dev->memory());
            if (_host_stage_alias == nullptr) { // the cache's own buffer: looked up once
                _host_stage_alias = kernels::mapped_host_alias(_host_stage->memory(), _host_stage->size());
            }
            if (q_by_kernel && aligned(_host_stage_alias)) {
                const void *src[2] = {_host_stage_alias, q_alias};
                void *dst[2] = {idx, q_d};
                const size_t bytes[2] = {idx_bytes, q_bytes};
                kernels::small_copies(stream, src, dst, bytes, 2);
            } else {
                api->memcpy_async(idx, idx_host, idx_bytes, LLAISYS_MEMCPY_H2D, stream);
                api->memcpy_async(q_d, q_host, q_bytes, LLAISYS_MEMCPY_H2D, stream);
            }
            // a plain launch: the kernel reads the index arrays before any wait, and they come from the launch before it
            launchDecode(layer, out_dst, nullptr, q_d, k_src, v_src, idx, idx + n_seqs, n_seqs, max_kv, nh, scale, stream, false);
        }
        if (out_dst == out_d) {
            api->memcpy_async(out_host, out_d, q_bytes, LLAISYS_MEMCPY_D2H, stream);
        }
        api->stream_synchronize(stream);
        return;
    }
#endif
    // every other pool (f32, other head dims or page sizes): plain copies, the append kernel, the generic attention kernel
    const int32_t *arrays[3] = {seq_ids, pos.data(), kv_lens};
    const size_t lens[3] = {n_seqs, n_seqs, n_seqs};
    int32_t *idx = stage(arrays, lens, 3);
    api->memcpy_async(k_d, k_new_host, kv_bytes, LLAISYS_MEMCPY_H2D, stream);
    api->memcpy_async(v_d, v_new_host, kv_bytes, LLAISYS_MEMCPY_H2D, stream);
    api->memcpy_async(q_d, q_host, q_bytes, LLAISYS_MEMCPY_H2D, stream);
    appendDev(layer, k_d, v_d, idx, idx + n_seqs, n_seqs, stream);
    decodeDev(layer, out_d, nullptr, q_d, idx, idx + 2 * n_seqs, n_seqs, max_kv, nh, scale, stream);
    api->memcpy_async(out_host, out_d, q_bytes, LLAISYS_MEMCPY_D2H, stream);
    api->stream_synchronize(stream);
}

void PagedKV::prefill(size_t layer, void *out, const void *q, const int32_t *seq_ids, const int32_t *q_lens,
                      const int32_t *kv_lens, size_t n_seqs, size_t nh, float scale) {
    checkLayer(layer);
    if (n_seqs == 0) {
        return;
    }
    KV_REQUIRE(seq_ids && q_lens && kv_lens, LLAISYS_E_INVALID, "paged attention: null index array");
    std::vector<int32_t> starts(n_seqs + 1, 0);
    size_t max_kv = 0, max_q = 0;
    for (size_t i = 0; i < n_seqs; ++i) {
        const Seq &s = liveSeq(seq_ids[i]);
        KV_REQUIRE(q_lens[i] >= 0 && kv_lens[i] >= q_lens[i], LLAISYS_E_INVALID,
                   "paged attention: sequence ", i, " has q_len ", q_lens[i], " > kv_len ", kv_lens[i]);
        KV_REQUIRE(size_t(kv_lens[i]) <= size_t(s.n_pages) * _cfg.page_size, LLAISYS_E_INVALID,
                   "paged attention: kv_len ", kv_lens[i], " exceeds the ", s.n_pages,
                   " page(s) reserved for sequence ", seq_ids[i]);
        KV_REQUIRE(size_t(starts[i]) + size_t(q_lens[i]) <= kMaxInt32, LLAISYS_E_INVALID, "paged attention: too many rows");
        starts[i + 1] = starts[i] + q_lens[i];
        max_kv = std::max(max_kv, size_t(kv_lens[i]));
        max_q = std::max(max_q, size_t(q_lens[i]));
    }
    const size_t total_q = size_t(starts[n_seqs]);
    flush();
    if (!onDevice()) {
        return prefillDev(layer, out, q, seq_ids, starts.data(), kv_lens, n_seqs, total_q, max_q, max_kv, nh, scale,
                          nullptr);
    }
    const int32_t *arrays[3] = {seq_ids, kv_lens, starts.data()};
    const size_t lens[3] = {n_seqs, n_seqs, n_seqs + 1};
    int32_t *dev = stage(arrays, lens, 3);
    prefillDev(layer, out, q, dev, dev + 2 * n_seqs, dev + n_seqs, n_seqs, total_q, max_q, max_kv, nh, scale,
               enter().stream());
}

// ---- kernel choice on NVIDIA ------------------------------------------------------------------------

namespace {
thread_local int g_last_attention_kernel = LLAISYS_KERNEL_NONE;
} // namespace

int lastAttentionKernel() { return g_last_attention_kernel; }
void noteAttentionKernel(int id) { g_last_attention_kernel = id; }

#ifdef ENABLE_NVIDIA_API
namespace {
// The shapes the specialised kernels are written for: 16-bit K/V, head_dim 128, 16-token pages, at most 8 query
// heads per kv head. Inside this domain a kernel that cannot take a call makes the call fail; it never hands the
// call to the generic kernel behind the caller's back.
bool fast_shape(llaisysDataType_t dtype, const kernels::KVView &view, const kernels::AttnBatch &batch) {
    return (dtype == LLAISYS_DTYPE_BF16 || dtype == LLAISYS_DTYPE_F16) && view.d == 128 && view.page_size == 16 &&
           view.nkvh > 0 && batch.nh % view.nkvh == 0 && batch.nh / view.nkvh <= 8;
}
} // namespace

int run_attention_nvidia(llaisysStream_t stream, llaisysDataType_t dtype, const kernels::KVView &view,
                         const kernels::AttnBatch &batch, const void *q, float scale, const kernels::AttnOut &out,
                         const kernels::AttnScratch &scratch) {
    const bool one_query_each = batch.q_starts == nullptr && batch.const_q_len == 1;
    const bool fast = fast_shape(dtype, view, batch);
    int used = LLAISYS_KERNEL_GENERIC;
    if (fast && one_query_each && view.block_table != nullptr && batch.kv_lens != nullptr) {
        // a page pool: the TMA kernel, or nothing
        const char *why = nullptr;
        if (kernels::attention_decode_tma(stream, dtype, view, batch, q, scale, out, scratch, nullptr, nullptr, &why) != 0) {
            fail(LLAISYS_E_UNSUPPORTED, "paged decode attention (TMA kernel): ", why ? why : "call not covered");
        }
        used = LLAISYS_KERNEL_DECODE_TMA;
    } else if (fast && one_query_each) {
        // one query over plain K/V tensors (the legacy operator): the cp.async split-KV kernel
        if (kernels::attention_decode_split(stream, dtype, view, batch, q, scale, out, scratch) != 0) {
            fail(LLAISYS_E_UNSUPPORTED, "decode attention (cp.async kernel): K/V, q or the scratch are not 16-byte aligned, "
                                        "or more than 1024 sequences");
        }
        used = LLAISYS_KERNEL_DECODE_CP_ASYNC;
    } else if (fast && out.part == nullptr &&
               (batch.q_starts != nullptr || (view.block_table == nullptr && batch.const_q_len >= 16))) {
        // chunks over a page pool, or the legacy operator's multi-token query over plain K/V tensors (from 16 rows on:
        // below that the 128-row tensor-core tile is mostly padding and the generic kernel serves the call)
        if (kernels::attention_prefill_tc(stream, dtype, view, batch, q, scale, out, scratch) != 0) {
            fail(LLAISYS_E_UNSUPPORTED, "chunk attention (tcgen05 kernel): q, out or K/V are not 16-byte aligned, the pool "
                                        "has no tensor map, or the workspace is missing");
        }
        used = LLAISYS_KERNEL_PREFILL_TC;
    } else {
        // f32 data, other head dims, page sizes or group widths, and short multi-token queries of the legacy operator
        kernels::attention_generic(stream, dtype, view, batch, q, scale, out, scratch.error_flag);
    }
    g_last_attention_kernel = used;
    return used;
}
#endif

} // namespace llaisys::kv
