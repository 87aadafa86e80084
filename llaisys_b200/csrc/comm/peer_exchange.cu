#include "peer_exchange.hpp"

#include "../kernels/device_utils.cuh"
#include "../kv/paged_kv.hpp"
#include "llaisys/paged_kv.h"

#include <algorithm>
#include <cstring>
#include <string>

namespace llaisys::comm {

namespace {

[[noreturn]] void fail(int code, const std::string &msg) { throw kv::StatusError(code, msg); }

void cuda_ok(cudaError_t rc, const char *what) {
    if (rc != cudaSuccess) {
        (void)cudaGetLastError();
        fail(LLAISYS_E_DEVICE, std::string(what) + ": " + cudaGetErrorString(rc));
    }
}

constexpr int kErrPeerTimeout = 1;

struct PeerTable {
    unsigned char *base[kMaxPeers]; // every rank's buffer as this rank sees it
};

// A slot word: a float and the step it belongs to, written and read as ONE aligned 8-byte access, so the two always
// travel together. The step is the word's own flag (the scheme of low-latency collectives): no fence orders anything.
__device__ __forceinline__ void store_word(uint2 *addr, float value, uint32_t step) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};\n" ::"l"(addr), "r"(__float_as_uint(value)), "r"(step) : "memory");
}
__device__ __forceinline__ uint2 load_word(const uint2 *addr) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(addr) : "memory");
    return v;
}

// For pools the TMA decode kernel does not serve: the partial was written locally as plain floats; one CTA per
// destination rank forwards it as slot words into slot `rank` (of the step's parity) of that rank's buffer.
__global__ void peer_push_kernel(PeerTable t, const float *__restrict__ src, size_t n_floats, size_t slot_floats, int rank,
                                 int world, size_t epoch_offset) {
    const uint32_t step = *reinterpret_cast<const uint32_t *>(t.base[rank] + epoch_offset) + 1;
    uint2 *dst = reinterpret_cast<uint2 *>(t.base[blockIdx.x]) + (size_t(step & 1u) * world + rank) * slot_floats;
    for (size_t i = threadIdx.x; i < n_floats; i += blockDim.x) {
        store_word(dst + i, src[i], step);
    }
}

// The value of a slot word once it carries `step`; polls (bounded) until it does. After one wait has run out the lane
// stops waiting: the step is lost anyway, and the kernel must end.
__device__ __forceinline__ float wait_word(const uint2 *addr, uint32_t step, uint32_t limit, bool &gave_up, int *error_word) {
    uint2 w = load_word(addr);
    uint32_t spins = 0;
    while (w.y != step && !gave_up) {
        if (++spins > limit) {
            gave_up = true;
            atomicOr(error_word, kErrPeerTimeout);
            break;
        }
        __nanosleep(100);
        w = load_word(addr);
    }
    return __uint_as_float(w.x);
}

// Merges every rank's slot: out[r] = sum_p w_p o_p[r] / sum_p w_p with w_p = l_p exp(m_p - M) (the same arithmetic, in
// the same order, as the library's LSE merge; one warp per row). Each value is taken when its word carries the step.
template <typename T>
__global__ void peer_merge_kernel(T *__restrict__ out, unsigned char *local_base, size_t slot_floats, int world, int n_rows,
                                  int d, size_t epoch_offset, size_t error_offset, uint32_t spin_limit) {
    // Launched with programmatic stream serialisation behind the decode kernel that feeds it: it starts while that kernel
    // still runs (its CTAs take SM slots the decode grid leaves free), takes values as they arrive, and lets its own
    // successor -- the next round's decode kernel -- start its page copies in turn.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const uint32_t step = *reinterpret_cast<const uint32_t *>(local_base + epoch_offset) + 1;
    int *error_word = reinterpret_cast<int *>(local_base + error_offset);
    const int warps_per_block = blockDim.x >> 5;
    const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    bool gave_up = false;
    if (row < n_rows) {
        const uint2 *parts = reinterpret_cast<const uint2 *>(local_base) + size_t(step & 1u) * world * slot_floats;
        const uint2 *base = parts + size_t(row) * (d + 2);
        // Every word a lane needs in one batch (4 dims x 8 ranks) is REQUESTED before any of them is looked at, and a
        // batch with a word still missing is asked for again as a whole: a word that has arrived costs one round trip to
        // L2 whether it is asked for alone or with thirty others, and taking them one after the other made the merge of
        // eight ranks' rows cost thirty-four such trips in a row.
        // (m, l) of every rank: lane p fetches rank p's pair, the warp shares them
        float m_mine = -INFINITY, l_mine = 0.f;
        if (lane < world) {
            const uint2 *at = base + size_t(lane) * slot_floats + d;
            const uint2 wm = load_word(at), wl = load_word(at + 1);
            m_mine = wm.y == step ? __uint_as_float(wm.x) : wait_word(at, step, spin_limit, gave_up, error_word);
            l_mine = wl.y == step ? __uint_as_float(wl.x) : wait_word(at + 1, step, spin_limit, gave_up, error_word);
        }
        __syncwarp();
        float m_all = -INFINITY;
        for (int p = 0; p < world; ++p) {
            const float l = __shfl_sync(0xffffffffu, l_mine, p), m = __shfl_sync(0xffffffffu, m_mine, p);
            if (l > 0.f) {
                m_all = fmaxf(m_all, m);
            }
        }
        float l_all = 0.f;
        for (int p = 0; p < world; ++p) {
            const float l = __shfl_sync(0xffffffffu, l_mine, p), m = __shfl_sync(0xffffffffu, m_mine, p);
            if (l > 0.f) {
                l_all += l * expf(m - m_all);
            }
        }
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        constexpr int kDimsAtOnce = 4, kRanksAtOnce = 8;
        for (int dim_first = 0; dim_first < d; dim_first += kDimsAtOnce * 32) { // uniform trip counts: shuffles inside
            float o[kDimsAtOnce];
#pragma unroll
            for (int a = 0; a < kDimsAtOnce; ++a) {
                o[a] = 0.f;
            }
            for (int p_first = 0; p_first < world; p_first += kRanksAtOnce) {
                float weight[kRanksAtOnce]; // 0 for a rank that saw no key (its words are not waited for) and past the last rank
#pragma unroll
                for (int b = 0; b < kRanksAtOnce; ++b) {
                    const int p = min(p_first + b, world - 1);
                    const float l = __shfl_sync(0xffffffffu, l_mine, p), m = __shfl_sync(0xffffffffu, m_mine, p);
                    weight[b] = (p_first + b < world && l > 0.f) ? l * expf(m - m_all) : 0.f;
                }
                uint2 w[kDimsAtOnce][kRanksAtOnce];
                for (uint32_t spins = 0;;) {
                    bool missing = false;
#pragma unroll
                    for (int a = 0; a < kDimsAtOnce; ++a) {
#pragma unroll
                        for (int b = 0; b < kRanksAtOnce; ++b) {
                            const int dim = dim_first + a * 32 + lane;
                            w[a][b] = make_uint2(0u, step);
                            if (dim < d && weight[b] != 0.f) {
                                w[a][b] = load_word(base + size_t(p_first + b) * slot_floats + dim);
                            }
                        }
                    }
#pragma unroll
                    for (int a = 0; a < kDimsAtOnce; ++a) {
#pragma unroll
                        for (int b = 0; b < kRanksAtOnce; ++b) {
                            missing = missing || w[a][b].y != step;
                        }
                    }
                    if (!missing || gave_up) {
                        break;
                    }
                    if (++spins > spin_limit) {
                        gave_up = true;
                        atomicOr(error_word, kErrPeerTimeout);
                        break;
                    }
                    __nanosleep(100);
                }
                // ranks in their order, one chain per dim: the sums are those of the library's LSE merge
#pragma unroll
                for (int b = 0; b < kRanksAtOnce; ++b) {
#pragma unroll
                    for (int a = 0; a < kDimsAtOnce; ++a) {
                        if (weight[b] != 0.f) {
                            o[a] = fmaf(weight[b], __uint_as_float(w[a][b].x), o[a]);
                        }
                    }
                }
            }
#pragma unroll
            for (int a = 0; a < kDimsAtOnce; ++a) {
                const int dim = dim_first + a * 32 + lane;
                if (dim < d) {
                    out[size_t(row) * d + dim] = kernels::from_f32<T>(o[a] * inv);
                }
            }
        }
    }
    // Completion of this kernel must imply completion of the decode kernel before it (its successor relies on that for
    // the scratch the two decode launches share): wait for it here, where nearly always it has long finished.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // The CTA that finishes last moves the step counter on (every CTA read it at its start, before it could finish).
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t *done = reinterpret_cast<uint32_t *>(local_base + epoch_offset) + 1;
        __threadfence();
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *done = 0;
            *reinterpret_cast<volatile uint32_t *>(local_base + epoch_offset) = step;
        }
    }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

} // namespace

PeerExchange::PeerExchange(int rank, int world, size_t slot_floats) : _rank(rank), _world(world), _slot_floats(slot_floats) {
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || slot_floats == 0 || slot_floats % 4 != 0) {
        fail(LLAISYS_E_INVALID, "peer exchange: bad rank, world size (at most 16) or slot size (a multiple of 4 floats)");
    }
    const size_t slots_bytes = 2 * size_t(world) * slot_floats * sizeof(uint2); // a word per float: value and step
    _epoch_offset = align_up(slots_bytes, 256);
    _error_offset = _epoch_offset + 256;
    _table_offset = _error_offset + 256; // every rank's buffer as THIS rank maps it (read by the decode kernel)
    _bytes = _table_offset + align_up(size_t(kMaxPeers) * sizeof(void *), 256);
    cuda_ok(cudaMalloc(&_base, _bytes), "peer exchange: cudaMalloc");
    cuda_ok(cudaMemset(_base, 0, _bytes), "peer exchange: cudaMemset");
    cuda_ok(cudaMalloc(&_local_part, slot_floats * sizeof(float)), "peer exchange: cudaMalloc");
    cuda_ok(cudaMemset(_local_part, 0, slot_floats * sizeof(float)), "peer exchange: cudaMemset");
    cuda_ok(cudaDeviceSynchronize(), "peer exchange: synchronize");
    _peer.assign(size_t(world), nullptr);
    _peer[size_t(rank)] = _base;
    _connected = world == 1;
    if (_connected) {
        writeTable();
    }
}

void PeerExchange::disconnect() {
    (void)cudaDeviceSynchronize();
    for (int p = 0; p < _world; ++p) {
        if (p != _rank && _peer[size_t(p)] != nullptr) {
            (void)cudaIpcCloseMemHandle(_peer[size_t(p)]);
            _peer[size_t(p)] = nullptr;
        }
    }
    (void)cudaGetLastError();
    _connected = false;
}

PeerExchange::~PeerExchange() {
    disconnect();
    (void)cudaFree(_local_part);
    (void)cudaFree(_base);
    (void)cudaGetLastError();
}

void PeerExchange::localHandle(void *out_64_bytes) const {
    static_assert(sizeof(cudaIpcMemHandle_t) == kIpcHandleBytes, "IPC handle size");
    if (out_64_bytes == nullptr) {
        fail(LLAISYS_E_INVALID, "peer exchange: null output");
    }
    cudaIpcMemHandle_t h;
    cuda_ok(cudaIpcGetMemHandle(&h, _base), "peer exchange: cudaIpcGetMemHandle");
    memcpy(out_64_bytes, &h, sizeof(h));
}

void PeerExchange::connect(const void *handles) {
    if (handles == nullptr) {
        fail(LLAISYS_E_INVALID, "peer exchange: null handles");
    }
    if (_connected) {
        fail(LLAISYS_E_INVALID, "peer exchange: already connected");
    }
    for (int p = 0; p < _world; ++p) {
        if (p == _rank) {
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const unsigned char *>(handles) + size_t(p) * kIpcHandleBytes, sizeof(h));
        void *mapped = nullptr;
        cuda_ok(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess), "peer exchange: cudaIpcOpenMemHandle");
        _peer[size_t(p)] = static_cast<unsigned char *>(mapped);
    }
    writeTable();
    _connected = true;
}

void PeerExchange::writeTable() {
    cuda_ok(cudaMemcpy(_base + _table_offset, _peer.data(), size_t(_world) * sizeof(unsigned char *), cudaMemcpyHostToDevice),
            "peer exchange: cudaMemcpy");
}

kernels::PeerSink PeerExchange::sink() const {
    if (!_connected) {
        fail(LLAISYS_E_INVALID, "peer exchange: connect() has not been called");
    }
    kernels::PeerSink k;
    k.table = reinterpret_cast<unsigned char *const *>(_base + _table_offset);
    k.own = _base;
    k.rows = _local_part;
    k.world = _world;
    k.rank = _rank;
    k.slot_floats = _slot_floats;
    k.epoch_offset = _epoch_offset;
    return k;
}

void PeerExchange::setWaitLimit(uint32_t polls) {
    if (polls == 0) {
        fail(LLAISYS_E_INVALID, "peer exchange: the wait limit must be at least one poll");
    }
    _spin_limit = polls;
}

void PeerExchange::push(llaisysStream_t stream, int n_rows, int d) {
    if (!_connected) {
        fail(LLAISYS_E_INVALID, "peer exchange: connect() has not been called");
    }
    if (n_rows <= 0 || d <= 0 || size_t(n_rows) * size_t(d + 2) > _slot_floats || (size_t(n_rows) * size_t(d + 2)) % 4 != 0) {
        fail(LLAISYS_E_INVALID, "peer exchange: rows do not fit the slot (or are not a multiple of 16 bytes)");
    }
    PeerTable t{};
    for (int p = 0; p < _world; ++p) {
        t.base[p] = _peer[size_t(p)];
    }
    peer_push_kernel<<<unsigned(_world), 512, 0, static_cast<cudaStream_t>(stream)>>>(
        t, _local_part, size_t(n_rows) * size_t(d + 2), _slot_floats, _rank, _world, _epoch_offset);
    kernels::check_launch("peer_exchange push");
}

void PeerExchange::merge(llaisysStream_t stream, llaisysDataType_t dtype, void *out, int n_rows, int d) {
    if (!_connected) {
        fail(LLAISYS_E_INVALID, "peer exchange: connect() has not been called");
    }
    if (n_rows <= 0 || d <= 0 || out == nullptr || size_t(n_rows) * size_t(d + 2) > _slot_floats) {
        fail(LLAISYS_E_INVALID, "peer exchange: rows do not fit the slot");
    }
    const int block = 128, grid = (n_rows + 3) / 4;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(unsigned(block));
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    auto go = [&](auto kernel, auto *typed_out) {
        cuda_ok(cudaLaunchKernelEx(&cfg, kernel, typed_out, _base, _slot_floats, _world, n_rows, d, _epoch_offset, _error_offset,
                                   _spin_limit),
                "peer exchange: merge launch");
    };
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        go(peer_merge_kernel<float>, static_cast<float *>(out));
        break;
    case LLAISYS_DTYPE_F16:
        go(peer_merge_kernel<__half>, static_cast<__half *>(out));
        break;
    case LLAISYS_DTYPE_BF16:
        go(peer_merge_kernel<__nv_bfloat16>, static_cast<__nv_bfloat16 *>(out));
        break;
    default:
        fail(LLAISYS_E_INVALID, "peer exchange: unsupported output type");
    }
    kernels::check_launch("peer_exchange merge");
}

int PeerExchange::status(llaisysStream_t stream) {
    auto s = static_cast<cudaStream_t>(stream);
    int host = 0;
    cuda_ok(cudaMemcpyAsync(&host, _base + _error_offset, sizeof(host), cudaMemcpyDeviceToHost, s), "peer exchange: status");
    cuda_ok(cudaStreamSynchronize(s), "peer exchange: status");
    if (host != 0) {
        cuda_ok(cudaMemsetAsync(_base + _error_offset, 0, sizeof(host), s), "peer exchange: status");
    }
    return host;
}

} // namespace llaisys::comm
