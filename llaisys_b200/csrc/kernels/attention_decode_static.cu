// llaisysPagedAttentionDecodeNoAlloc: the split-KV decode for callers that must not allocate device memory.
//
// Who that is: a serving process that hands every free byte of HBM to its own page pool at start-up (a later
// cudaMalloc from a library then fails, or fragments what the server wanted contiguous), and a latency-bound
// decode loop in which an allocation or release would stall the whole device (cudaFree waits for all streams).
// Such a caller owns the page pool, the block tables and the query/output buffers already; the only thing the
// decode kernel needs beyond them is scratch for the split-KV partial results and arrival counters. Here that
// scratch is a fixed array in the library's device image, so the call touches no allocator at all.
//
// Consequences the caller has to know:
//   * the array has a fixed size: n_seqs * nkvh <= kMaxPairs and a GPU of at most kMaxCtas / 2 SMs; anything larger
//     is refused with LLAISYS_E_INVALID before any work is queued;
//   * every GPU that loads the library carries the array (about 3.5 MiB) until the process exits;
//   * all calls on a device share it. The arrival counters are cleared at the start of every call; the partials need
//     no clearing (each launch writes a slot before reading it). Two calls that overlap on the GPU -- different
//     streams, no ordering between them -- race on it and give garbage: keep calls on one device ordered;
//   * the first call on each device resolves the array's device address (cudaGetSymbolAddress). Make that first
//     call outside any stream capture; a call whose look-up fails reports it and the next call tries again;
//   * a caller that passes no error word of its own gets the kernel's "skipped a bad page" bits collected in a word
//     inside the array, which stays set until llaisysPagedAttentionDecodeNoAllocStatus reads and clears it;
//   * the call runs with device_id current and puts the caller's current device back before it returns.
#include "kernels.hpp"
#include "device_utils.cuh"

#include "llaisys/paged_kv.h"

#include <mutex>
#include <string>

namespace {

constexpr int kMaxPairs = 512;      // n_seqs * nkvh per call
constexpr int kMaxCtas = 320;       // persistent CTAs of the decode kernel: two per SM, up to 160 SMs
constexpr int kMaxGroup = 8;        // query heads per kv head
constexpr int kPartStride = 132;    // floats per (slot, head) partial
constexpr size_t kPartialFloats = size_t(kMaxCtas + kMaxPairs) * kMaxGroup * kPartStride;
constexpr int kMaxDevices = 64;

struct StaticScratch {
    float partials[kPartialFloats];
    int32_t counters[kMaxPairs];
    int32_t error_word;
};

// The name below is a host-side handle only; its device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) StaticScratch g_decode_scratch;

struct DeviceSlot {
    std::mutex lock;
    StaticScratch *ptr = nullptr; // set once the look-up has succeeded; a failed look-up is retried by the next call
};
DeviceSlot g_slots[kMaxDevices];

// Makes `device` current for the life of the object and the previous device current again afterwards.
struct DeviceScope {
    int previous = -1;
    explicit DeviceScope(int device) {
        LLAISYS_CUDA_CHECK(cudaGetDevice(&previous));
        if (previous != device) {
            LLAISYS_CUDA_CHECK(cudaSetDevice(device));
        } else {
            previous = -1;
        }
    }
    ~DeviceScope() {
        if (previous >= 0 && cudaSetDevice(previous) != cudaSuccess) {
            (void)cudaGetLastError();
        }
    }
};

// Device address of the static array on the CURRENT device; throws if the runtime cannot give it (nothing is cached then).
StaticScratch *scratch_of(int device_id) {
    DeviceSlot &slot = g_slots[device_id];
    std::lock_guard<std::mutex> guard(slot.lock);
    if (slot.ptr == nullptr) {
        void *p = nullptr;
        LLAISYS_CUDA_CHECK(cudaGetSymbolAddress(&p, g_decode_scratch));
        slot.ptr = static_cast<StaticScratch *>(p);
    }
    return slot.ptr;
}

} // namespace

namespace llaisys::kernels {
// Lets llaisysGetLastError report this file's message (defined in capi/paged_kv.cc).
void set_last_error(const std::string &msg);
} // namespace llaisys::kernels

extern "C" LLAISYS_API int llaisysPagedAttentionDecodeNoAlloc(
    int device_id, void *out, const void *q, void *pool_layer, const int32_t *block_table_dev, size_t table_stride,
    size_t num_pages, const int32_t *seq_ids_dev, const int32_t *kv_lens_dev, size_t n_seqs, size_t max_kv_len, size_t nh,
    size_t nkvh, llaisysDataType_t dtype, float scale, int32_t *error_flag_dev, llaisysStream_t stream) {
    using namespace llaisys::kernels;
    auto report = [](int code, const std::string &msg) {
        set_last_error(msg);
        return code;
    };
    if (n_seqs == 0) {
        return LLAISYS_OK;
    }
    if (out == nullptr || q == nullptr || pool_layer == nullptr || block_table_dev == nullptr || kv_lens_dev == nullptr) {
        return report(LLAISYS_E_INVALID, "decode (no-alloc): null pointer argument");
    }
    if (dtype != LLAISYS_DTYPE_BF16 && dtype != LLAISYS_DTYPE_F16) {
        return report(LLAISYS_E_UNSUPPORTED, "decode (no-alloc): K/V must be BF16 or F16 (head_dim 128, 16-token pages)");
    }
    if (nkvh == 0 || nh == 0 || nh % nkvh != 0 || nh / nkvh > size_t(kMaxGroup)) {
        return report(LLAISYS_E_INVALID, "decode (no-alloc): nh must be a multiple of nkvh with at most 8 query heads per kv head");
    }
    if (n_seqs * nkvh > size_t(kMaxPairs)) {
        return report(LLAISYS_E_INVALID, "decode (no-alloc): n_seqs * nkvh = " + std::to_string(n_seqs * nkvh) +
                                             " exceeds the static scratch limit of " + std::to_string(kMaxPairs) +
                                             "; use llaisysPagedAttentionDecodeDev or split the batch");
    }
    if (num_pages == 0 || num_pages > size_t(INT32_MAX) || table_stride == 0 || table_stride * 16 > size_t(INT32_MAX) ||
        max_kv_len > table_stride * 16) {
        return report(LLAISYS_E_INVALID, "decode (no-alloc): page pool / block table sizes out of range");
    }
    if (device_id < 0 || device_id >= kMaxDevices) {
        return report(LLAISYS_E_INVALID, "decode (no-alloc): device id out of range");
    }
    try {
        DeviceScope scope(device_id);
        // set-up, once per device, with that device current: the device address of the static array
        StaticScratch *scratch = scratch_of(device_id);
        const int grid = decode_grid_size(int32_t(n_seqs), int32_t(nkvh), int32_t(max_kv_len));
        if (grid > kMaxCtas) {
            return report(LLAISYS_E_INVALID, "decode (no-alloc): this GPU has more SMs than the static scratch was sized for");
        }
        auto s = static_cast<cudaStream_t>(stream);
        // the arrival counters must start at zero; a call that was cut short may have left some set
        LLAISYS_CUDA_CHECK(cudaMemsetAsync(scratch->counters, 0, sizeof(scratch->counters), s));

        KVView kv;
        const size_t tile = 16 * 128; // elements of one (page, K|V, kv-head) tile
        kv.k_base = pool_layer;
        kv.v_base = static_cast<char *>(pool_layer) + nkvh * tile * 2;
        kv.page_stride = int64_t(2 * nkvh * tile);
        kv.head_stride = int64_t(tile);
        kv.token_stride = 128;
        kv.block_table = block_table_dev;
        kv.table_stride = int32_t(table_stride);
        kv.page_size = 16;
        kv.num_pages = int32_t(num_pages);
        kv.nkvh = int32_t(nkvh);
        kv.d = 128;
        AttnBatch batch;
        batch.seq_ids = seq_ids_dev;
        batch.kv_lens = kv_lens_dev;
        batch.const_q_len = 1;
        batch.n_seqs = int32_t(n_seqs);
        batch.total_q = int32_t(n_seqs);
        batch.max_q_len = 1;
        batch.max_kv_len = int32_t(max_kv_len);
        batch.nh = int32_t(nh);
        AttnOut o;
        o.out = out;
        AttnScratch sc;
        sc.partials = scratch->partials;
        sc.partials_floats = kPartialFloats;
        sc.counters = scratch->counters;
        sc.counters_len = kMaxPairs;
        sc.error_flag = error_flag_dev != nullptr ? error_flag_dev : &scratch->error_word;
        if (attention_decode_split(stream, dtype, kv, batch, q, scale, o, sc) != 0) {
            return report(LLAISYS_E_UNSUPPORTED, "decode (no-alloc): shape not covered by the split-KV kernel "
                                                 "(needs 16-byte aligned pool and q, n_seqs <= 1024)");
        }
        return LLAISYS_OK;
    } catch (const std::exception &e) {
        return report(LLAISYS_E_DEVICE, e.what());
    }
}

// Reads (and clears) the error bits that calls WITHOUT an error word of their own have collected on the device since
// the last read. Synchronises `stream` first; allocates nothing.
extern "C" LLAISYS_API int llaisysPagedAttentionDecodeNoAllocStatus(int device_id, llaisysStream_t stream,
                                                                    int32_t *flags_out) {
    using namespace llaisys::kernels;
    if (flags_out == nullptr || device_id < 0 || device_id >= kMaxDevices) {
        set_last_error("decode (no-alloc) status: bad device id or null output");
        return LLAISYS_E_INVALID;
    }
    try {
        DeviceScope scope(device_id);
        StaticScratch *scratch = scratch_of(device_id);
        auto s = static_cast<cudaStream_t>(stream);
        LLAISYS_CUDA_CHECK(cudaMemcpyAsync(flags_out, &scratch->error_word, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
        LLAISYS_CUDA_CHECK(cudaStreamSynchronize(s));
        if (*flags_out != 0) {
            LLAISYS_CUDA_CHECK(cudaMemsetAsync(&scratch->error_word, 0, sizeof(int32_t), s));
        }
        return LLAISYS_OK;
    } catch (const std::exception &e) {
        set_last_error(e.what());
        return LLAISYS_E_DEVICE;
    }
}
