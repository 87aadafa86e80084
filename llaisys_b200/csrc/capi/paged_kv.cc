// extern "C" thunks of the paged-KV API. Unlike the legacy ABI these never let an exception out: every
// failure becomes a status code plus a thread-local message (llaisysGetLastError).
#include "llaisys/paged_kv.h"

#include "../comm/peer_exchange.hpp"
#include "../core/core.hpp"

#include "../cpu/cpu_kernels.hpp"
#include "../kv/paged_kv.hpp"
#ifdef ENABLE_NVIDIA_API
#include "../kernels/kernels.hpp"
#endif

#include <string>

struct LlaisysPagedKV {
    llaisys::kv::PagedKV impl;
    explicit LlaisysPagedKV(const llaisys::kv::PagedKVConfig &cfg) : impl(cfg) {}
};

namespace {

thread_local std::string g_last_error;

template <typename F>
int guarded(F &&body) {
    try {
        body();
        return LLAISYS_OK;
    } catch (const llaisys::kv::StatusError &e) {
        g_last_error = e.what();
        return e.code;
    } catch (const std::invalid_argument &e) {
        g_last_error = e.what();
        return LLAISYS_E_INVALID;
    } catch (const std::bad_alloc &) {
        g_last_error = "out of host memory";
        return LLAISYS_E_DEVICE;
    } catch (const std::exception &e) {
        g_last_error = e.what();
        return LLAISYS_E_DEVICE;
    } catch (...) {
        g_last_error = "unknown error";
        return LLAISYS_E_DEVICE;
    }
}

} // namespace

namespace llaisys::kernels {
// Entry points that live beside their kernels (attention_decode_static.cu) record their message here.
void set_last_error(const std::string &msg) { g_last_error = msg; }
} // namespace llaisys::kernels

namespace {

int null_handle() {
    g_last_error = "paged KV: null cache handle";
    return LLAISYS_E_INVALID;
}

} // namespace

#define KV_OR_FAIL(kv)        \
    if ((kv) == nullptr) {    \
        return null_handle(); \
    }

extern "C" {

const char *llaisysGetLastError(void) { return g_last_error.c_str(); }

int llaisysPagedKVCreate(llaisysPagedKV_t *kv_out, llaisysDeviceType_t device_type, int device_id,
                         llaisysDataType_t dtype, size_t nlayer, size_t num_pages, size_t page_size, size_t nkvh,
                         size_t head_dim, size_t max_seqs, size_t max_pages_per_seq) {
    return guarded([&] {
        if (kv_out == nullptr) {
            throw llaisys::kv::StatusError(LLAISYS_E_INVALID, "paged KV: kv_out is null");
        }
        *kv_out = nullptr;
        llaisys::kv::PagedKVConfig cfg;
        cfg.device_type = device_type;
        cfg.device_id = device_id;
        cfg.dtype = dtype;
        cfg.nlayer = nlayer;
        cfg.num_pages = num_pages;
        cfg.page_size = page_size;
        cfg.nkvh = nkvh;
        cfg.head_dim = head_dim;
        cfg.max_seqs = max_seqs;
        cfg.max_pages_per_seq = max_pages_per_seq;
        *kv_out = new LlaisysPagedKV(cfg);
    });
}

int llaisysPagedKVDestroy(llaisysPagedKV_t kv) {
    return guarded([&] { delete kv; });
}

int llaisysPagedKVSeqAdd(llaisysPagedKV_t kv, int32_t *seq_out) {
    KV_OR_FAIL(kv);
    return guarded([&] {
        if (seq_out == nullptr) {
            throw llaisys::kv::StatusError(LLAISYS_E_INVALID, "paged KV: seq_out is null");
        }
        *seq_out = kv->impl.seqAdd();
    });
}
int llaisysPagedKVSeqReserve(llaisysPagedKV_t kv, int32_t seq, size_t n_tokens) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.seqReserve(seq, n_tokens); });
}
int llaisysPagedKVSeqAssignPages(llaisysPagedKV_t kv, int32_t seq, const int32_t *pages, size_t n_pages) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.seqAssignPages(seq, pages, n_pages); });
}
int llaisysPagedKVSeqFree(llaisysPagedKV_t kv, int32_t seq) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.seqFree(seq); });
}
size_t llaisysPagedKVNumFreePages(llaisysPagedKV_t kv) { return kv ? kv->impl.numFreePages() : 0; }
size_t llaisysPagedKVNumSeqs(llaisysPagedKV_t kv) { return kv ? kv->impl.numSeqs() : 0; }
int64_t llaisysPagedKVSeqNumPages(llaisysPagedKV_t kv, int32_t seq) { return kv ? kv->impl.seqNumPages(seq) : -1; }
int llaisysPagedKVSeqPages(llaisysPagedKV_t kv, int32_t seq, int32_t *pages_out, size_t cap) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.seqPages(seq, pages_out, cap); });
}

void *llaisysPagedKVPoolData(llaisysPagedKV_t kv, size_t layer) {
    void *p = nullptr;
    if (kv != nullptr) {
        guarded([&] { p = kv->impl.poolData(layer); });
    }
    return p;
}
size_t llaisysPagedKVLayerBytes(llaisysPagedKV_t kv) { return kv ? kv->impl.layerBytes() : 0; }
const int32_t *llaisysPagedKVBlockTableData(llaisysPagedKV_t kv) { return kv ? kv->impl.blockTableData() : nullptr; }
int llaisysPagedKVSetLaunchOverlap(llaisysPagedKV_t kv, int enable) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.setLaunchOverlap(enable != 0); });
}
int llaisysPagedKVFlush(llaisysPagedKV_t kv) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.flush(); });
}
int llaisysPagedKVCheck(llaisysPagedKV_t kv) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.check(); });
}

int llaisysPagedKVAppend(llaisysPagedKV_t kv, size_t layer, const void *k_rows, const void *v_rows,
                         const int32_t *seq_ids, const int32_t *positions, size_t n_rows) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.append(layer, k_rows, v_rows, seq_ids, positions, n_rows); });
}
int llaisysPagedKVGather(llaisysPagedKV_t kv, size_t layer, int32_t seq, size_t n_tokens, void *k_out, void *v_out) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.gather(layer, seq, n_tokens, k_out, v_out); });
}
int llaisysPagedAttentionDecode(llaisysPagedKV_t kv, size_t layer, void *out, const void *q, const int32_t *seq_ids,
                                const int32_t *kv_lens, size_t n_seqs, size_t nh, float scale) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.decode(layer, out, nullptr, q, seq_ids, kv_lens, n_seqs, nh, scale); });
}
int llaisysPagedAttentionPrefill(llaisysPagedKV_t kv, size_t layer, void *out, const void *q, const int32_t *seq_ids,
                                 const int32_t *q_lens, const int32_t *kv_lens, size_t n_seqs, size_t nh,
                                 float scale) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.prefill(layer, out, q, seq_ids, q_lens, kv_lens, n_seqs, nh, scale); });
}
int llaisysPagedAttentionDecodePartial(llaisysPagedKV_t kv, size_t layer, float *part, const void *q,
                                       const int32_t *seq_ids, const int32_t *kv_lens, size_t n_seqs, size_t nh,
                                       float scale) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.decode(layer, nullptr, part, q, seq_ids, kv_lens, n_seqs, nh, scale); });
}

int llaisysLseMerge(llaisysDeviceType_t device_type, int device_id, void *out, llaisysDataType_t dtype,
                    const float *parts, size_t n_parts, size_t n_rows, size_t head_dim) {
    return guarded([&] {
        using llaisys::kv::StatusError;
        if (n_rows == 0 || head_dim == 0) {
            return;
        }
        if (out == nullptr || parts == nullptr || n_parts == 0) {
            throw StatusError(LLAISYS_E_INVALID, "lse merge: null argument or no parts");
        }
        if (n_parts > 65535 || n_rows > (size_t(1) << 30) || head_dim > 65535) {
            throw StatusError(LLAISYS_E_INVALID, "lse merge: sizes out of range");
        }
        if (dtype != LLAISYS_DTYPE_F32 && dtype != LLAISYS_DTYPE_F16 && dtype != LLAISYS_DTYPE_BF16) {
            throw StatusError(LLAISYS_E_INVALID, "lse merge: dtype must be F32, F16 or BF16");
        }
        if (device_type == LLAISYS_DEVICE_CPU) {
            llaisys::cpu::lse_merge(dtype, out, parts, int32_t(n_parts), int32_t(n_rows), int32_t(head_dim));
            return;
        }
#ifdef ENABLE_NVIDIA_API
        if (device_type == LLAISYS_DEVICE_NVIDIA) {
            auto &ctx = llaisys::core::context();
            ctx.setDevice(device_type, device_id);
            llaisys::kernels::lse_merge(ctx.runtime().stream(), dtype, out, parts, int32_t(n_parts), int32_t(n_rows),
                                        int32_t(head_dim));
            return;
        }
#endif
        throw StatusError(LLAISYS_E_UNSUPPORTED, "lse merge: unsupported device");
    });
}

int llaisysPagedDecodeStepHost(llaisysPagedKV_t kv, size_t layer, void *out_host, const void *q_host, const void *k_new_host,
                               const void *v_new_host, const int32_t *seq_ids, const int32_t *kv_lens, size_t n_seqs,
                               size_t nh, float scale) {
    KV_OR_FAIL(kv);
    return guarded([&] {
        kv->impl.decodeStepHost(layer, out_host, q_host, k_new_host, v_new_host, seq_ids, kv_lens, n_seqs, nh, scale);
    });
}

#ifdef ENABLE_NVIDIA_API
struct LlaisysPeerExchange {
    llaisys::comm::PeerExchange impl;
    int device_id;
    LlaisysPeerExchange(int device, int rank, int world, size_t slot_floats) : impl(rank, world, slot_floats), device_id(device) {}
};
#else
struct LlaisysPeerExchange {};
#endif

int llaisysPeerExchangeCreate(llaisysPeerExchange_t *ex_out, int device_id, int rank, int world, size_t slot_floats) {
    if (ex_out == nullptr) {
        llaisys::kernels::set_last_error("peer exchange: null output");
        return LLAISYS_E_INVALID;
    }
#ifdef ENABLE_NVIDIA_API
    return guarded([&] {
        llaisys::core::context().setDevice(LLAISYS_DEVICE_NVIDIA, device_id);
        *ex_out = new LlaisysPeerExchange(device_id, rank, world, slot_floats);
    });
#else
    (void)device_id, (void)rank, (void)world, (void)slot_floats;
    llaisys::kernels::set_last_error("this build has no NVIDIA backend");
    return LLAISYS_E_UNSUPPORTED;
#endif
}
void llaisysPeerExchangeDestroy(llaisysPeerExchange_t ex) {
#ifdef ENABLE_NVIDIA_API
    if (ex != nullptr) {
        try {
            llaisys::core::context().setDevice(LLAISYS_DEVICE_NVIDIA, ex->device_id);
        } catch (...) {
        }
    }
#endif
    delete ex;
}
#ifdef ENABLE_NVIDIA_API
#define EX_OR_FAIL(ex)                                                  \
    if ((ex) == nullptr) {                                              \
        llaisys::kernels::set_last_error("peer exchange: null handle"); \
        return LLAISYS_E_INVALID;                                       \
    }
int llaisysPeerExchangeHandle(llaisysPeerExchange_t ex, void *out_64_bytes) {
    EX_OR_FAIL(ex);
    return guarded([&] { ex->impl.localHandle(out_64_bytes); });
}
int llaisysPeerExchangeConnect(llaisysPeerExchange_t ex, const void *handles) {
    EX_OR_FAIL(ex);
    return guarded([&] {
        llaisys::core::context().setDevice(LLAISYS_DEVICE_NVIDIA, ex->device_id);
        ex->impl.connect(handles);
    });
}
int llaisysPagedAttentionDecodeSplitDev(llaisysPagedKV_t kv, size_t layer, void *out, const void *q, const int32_t *seq_ids_dev,
                                        const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len, size_t nh, float scale,
                                        llaisysPeerExchange_t ex, llaisysStream_t stream) {
    KV_OR_FAIL(kv);
    EX_OR_FAIL(ex);
    return guarded([&] {
        const auto &cfg = kv->impl.config();
        const size_t rows = n_seqs * nh;
        if (rows * (cfg.head_dim + 2) > ex->impl.slotFloats()) {
            throw llaisys::kv::StatusError(LLAISYS_E_INVALID, "split decode: the exchange's slots are too small for this batch");
        }
        if (kv->impl.canPushPartials(nh)) {
            // the decode kernel stores its rows at every rank and stamps the flags itself
            const llaisys::kernels::PeerSink sink = ex->impl.sink();
            kv->impl.decodeSplitDev(layer, q, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh, scale, sink, stream);
        } else {
            kv->impl.decodeDev(layer, nullptr, ex->impl.localPartial(), q, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh,
                               scale, stream);
            ex->impl.push(stream, int(rows), int(cfg.head_dim));
        }
        ex->impl.merge(stream, cfg.dtype, out, int(rows), int(cfg.head_dim));
    });
}
int llaisysPeerExchangeDisconnect(llaisysPeerExchange_t ex) {
    if (ex == nullptr) {
        g_last_error = "peer exchange: null handle";
        return LLAISYS_E_INVALID;
    }
    return guarded([&] { ex->impl.disconnect(); });
}
int llaisysPeerExchangeSetWaitLimit(llaisysPeerExchange_t ex, uint32_t polls) {
    if (ex == nullptr) {
        g_last_error = "peer exchange: null handle";
        return LLAISYS_E_INVALID;
    }
    return guarded([&] { ex->impl.setWaitLimit(polls); });
}
int llaisysPeerExchangeStatus(llaisysPeerExchange_t ex, llaisysStream_t stream) {
    if (ex == nullptr) {
        return -1;
    }
    int status = -1;
    const int rc = guarded([&] { status = ex->impl.status(stream); });
    return rc == LLAISYS_OK ? status : -1;
}
#else
int llaisysPeerExchangeHandle(llaisysPeerExchange_t, void *) { return LLAISYS_E_UNSUPPORTED; }
int llaisysPeerExchangeConnect(llaisysPeerExchange_t, const void *) { return LLAISYS_E_UNSUPPORTED; }
int llaisysPagedAttentionDecodeSplitDev(llaisysPagedKV_t, size_t, void *, const void *, const int32_t *, const int32_t *, size_t,
                                        size_t, size_t, float, llaisysPeerExchange_t, llaisysStream_t) {
    return LLAISYS_E_UNSUPPORTED;
}
int llaisysPeerExchangeDisconnect(llaisysPeerExchange_t) { return LLAISYS_E_UNSUPPORTED; }
int llaisysPeerExchangeSetWaitLimit(llaisysPeerExchange_t, uint32_t) { return LLAISYS_E_UNSUPPORTED; }
int llaisysPeerExchangeStatus(llaisysPeerExchange_t, llaisysStream_t) { return -1; }
#endif

int llaisysPagedKVSeqPublish(llaisysPagedKV_t kv, int32_t seq, const int64_t *tokens, size_t n_tokens) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.seqPublish(seq, tokens, n_tokens); });
}
int llaisysPagedKVSeqMatchPrefix(llaisysPagedKV_t kv, int32_t seq, const int64_t *tokens, size_t n_tokens,
                                 size_t *matched_out) {
    KV_OR_FAIL(kv);
    if (matched_out == nullptr) {
        llaisys::kernels::set_last_error("paged KV match: matched_out is null");
        return LLAISYS_E_INVALID;
    }
    return guarded([&] { *matched_out = kv->impl.seqMatchPrefix(seq, tokens, n_tokens); });
}
int llaisysPagedKVSeqFork(llaisysPagedKV_t kv, int32_t parent, size_t n_tokens, int32_t *child_out) {
    KV_OR_FAIL(kv);
    if (child_out == nullptr) {
        llaisys::kernels::set_last_error("paged KV fork: child_out is null");
        return LLAISYS_E_INVALID;
    }
    return guarded([&] { *child_out = kv->impl.seqFork(parent, n_tokens); });
}
int llaisysPagedKVPageRefCount(llaisysPagedKV_t kv, int32_t page) { return kv ? kv->impl.pageRefCount(page) : -1; }
size_t llaisysPagedKVNumCachedPages(llaisysPagedKV_t kv) { return kv ? kv->impl.numCachedPages() : 0; }

int llaisysPagedKVAppendDev(llaisysPagedKV_t kv, size_t layer, const void *k_rows, const void *v_rows,
                            const int32_t *seq_ids_dev, const int32_t *positions_dev, size_t n_rows,
                            llaisysStream_t stream) {
    KV_OR_FAIL(kv);
    return guarded([&] { kv->impl.appendDev(layer, k_rows, v_rows, seq_ids_dev, positions_dev, n_rows, stream); });
}
int llaisysPagedKVRopeAppendDev(llaisysPagedKV_t kv, size_t layer, void *q_out, const void *qkv, const void *bias,
                                const int32_t *seq_ids_dev, const int32_t *positions_dev, size_t n_rows, size_t nh,
                                float theta, llaisysStream_t stream) {
    KV_OR_FAIL(kv);
    return guarded(
        [&] { kv->impl.ropeAppendDev(layer, q_out, qkv, bias, seq_ids_dev, positions_dev, n_rows, nh, theta, stream); });
}
int llaisysPagedAttentionDecodeDev(llaisysPagedKV_t kv, size_t layer, void *out, const void *q,
                                   const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs,
                                   size_t max_kv_len, size_t nh, float scale, llaisysStream_t stream) {
    KV_OR_FAIL(kv);
    return guarded([&] {
        kv->impl.decodeDev(layer, out, nullptr, q, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh, scale, stream);
    });
}
int llaisysPagedDecodeStepDev(llaisysPagedKV_t kv, size_t layer, void *out, const void *q, const void *k_new,
                              const void *v_new, const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs,
                              size_t max_kv_len, size_t nh, float scale, llaisysStream_t stream) {
    KV_OR_FAIL(kv);
    return guarded([&] {
        kv->impl.decodeStepDev(layer, out, q, k_new, v_new, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh, scale, stream);
    });
}
int llaisysPagedKVLastKernel(llaisysPagedKV_t kv) { return kv ? kv->impl.lastKernel() : -1; }
int llaisysLastAttentionKernel(void) { return llaisys::kv::lastAttentionKernel(); }
int llaisysPagedAttentionDecodePartialDev(llaisysPagedKV_t kv, size_t layer, float *part, const void *q,
                                          const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs,
                                          size_t max_kv_len, size_t nh, float scale, llaisysStream_t stream) {
    KV_OR_FAIL(kv);
    return guarded([&] {
        kv->impl.decodeDev(layer, nullptr, part, q, seq_ids_dev, kv_lens_dev, n_seqs, max_kv_len, nh, scale, stream);
    });
}
int llaisysPagedAttentionPrefillDev(llaisysPagedKV_t kv, size_t layer, void *out, const void *q,
                                    const int32_t *seq_ids_dev, const int32_t *q_starts_dev,
                                    const int32_t *kv_lens_dev, size_t n_seqs, size_t total_q, size_t max_q_len,
                                    size_t max_kv_len, size_t nh, float scale, llaisysStream_t stream) {
    KV_OR_FAIL(kv);
    return guarded([&] {
        kv->impl.prefillDev(layer, out, q, seq_ids_dev, q_starts_dev, kv_lens_dev, n_seqs, total_q, max_q_len,
                            max_kv_len, nh, scale, stream);
    });
}

} // extern "C"
