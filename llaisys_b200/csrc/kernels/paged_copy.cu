// K1 paged append and K5 paged gather: bit-exact row movement between [rows, nkvh, d] tensors and the page
// pool, 16 bytes per thread.
//
// Work decomposition: one thread per 16-byte piece of one (row, K-or-V, kv-head) head-row. A head-row is
// d*elem_size bytes (256 B for bf16, d 128) and is contiguous on both sides, so a quarter-warp moves a full
// head-row with coalesced 128-bit loads and stores. The slot lookup (two int32 loads per row, then one table
// entry) hits in L1 for the other threads of the row.
//
// Roofline: HBM. Algorithmic bytes per row = 2 * (2 * nkvh * d * elem_size) (read the new K and V row, write
// them) + 8 (sequence id and position) + 4 (table entry).
#include "device_utils.cuh"
#include "kernels.hpp"

#include <algorithm>

namespace llaisys::kernels {

namespace {

struct CopyGeom {
    int64_t page_stride_b, head_stride_b, token_stride_b; // in bytes
    int32_t vecs_per_head_row;                            // d * elem_size / 16
    int32_t nkvh, page_size, num_pages, table_stride;
};

// Resolves (table row, position) to a physical page and slot; returns false (and flags) if out of range.
__device__ __forceinline__ bool resolve_slot(const int32_t *__restrict__ table, const CopyGeom &g, int32_t seq_row,
                                             int32_t pos, int32_t max_blocks, int32_t *error_flag, int32_t &page,
                                             int32_t &slot) {
    const int32_t blk = pos / g.page_size;
    if (pos < 0 || blk >= max_blocks || seq_row < 0) {
        atomicOr(error_flag, kErrBadPosition);
        return false;
    }
    page = table ? table[int64_t(seq_row) * g.table_stride + blk] : blk;
    slot = pos - blk * g.page_size;
    if (page < 0 || page >= g.num_pages) {
        atomicOr(error_flag, kErrBadPage);
        return false;
    }
    return true;
}

// One warp per new row, kRows rows per warp and pass. A row is moved by lane l as 16-byte piece l (+ 32, ...) of the K
// row and of the V row: with 2 kv-heads of 128 16-bit dims a row of K is 512 B, one coalesced warp-wide read, written as
// two 256 B head-rows. What bounds the kernel is latency, not bytes: a row's slot takes three dependent loads (sequence
// id and position, then the table entry), and with one row per warp in flight that chain -- not the 2 KiB moved -- set
// the pace (63 % of the copy rate). So a pass first issues the index loads AND the data loads of all its rows, which do
// not depend on the slots, then resolves the slots, then stores: kRows KiB of reads in flight per warp while the index
// chain runs underneath.
template <int kRows, int kIters>
__global__ void __launch_bounds__(256)
    paged_append_kernel(uint4 *__restrict__ k_pool, uint4 *__restrict__ v_pool, const uint4 *__restrict__ k_rows,
                        const uint4 *__restrict__ v_rows, const int32_t *__restrict__ table,
                        const int32_t *__restrict__ seq_ids, const int32_t *__restrict__ positions, CopyGeom g,
                        int32_t n_rows, int32_t max_blocks, int32_t *error_flag, const uint4 *__restrict__ side_src,
                        uint4 *__restrict__ side_dst, int32_t side_vecs) {
    // Under a programmatic launch this grid may start early: let the next kernel do the same, then wait for the
    // previous one (it may still be reading the pages this grid writes).
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int32_t vecs_per_row = g.vecs_per_head_row * g.nkvh; // per K (or V) row; at most 32 * kIters
    const int lane = threadIdx.x & 31;
    const int32_t warps = int32_t((gridDim.x * blockDim.x) >> 5);
    const int32_t warp_id = int32_t((blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    for (int32_t row0 = warp_id; row0 < n_rows; row0 += kRows * warps) {
        int32_t seq[kRows], pos[kRows];
        uint4 kd[kRows][kIters], vd[kRows][kIters];
#pragma unroll
        for (int u = 0; u < kRows; ++u) {
            const int32_t row = row0 + u * warps;
            seq[u] = row < n_rows ? seq_ids[row] : -1;
            pos[u] = row < n_rows ? positions[row] : 0;
        }
#pragma unroll
        for (int u = 0; u < kRows; ++u) {
            const int32_t row = row0 + u * warps;
#pragma unroll
            for (int it = 0; it < kIters; ++it) {
                const int32_t in_row = lane + 32 * it;
                if (row < n_rows && in_row < vecs_per_row) {
                    const int64_t src = int64_t(row) * vecs_per_row + in_row;
                    kd[u][it] = __ldcs(k_rows + src); // read once: do not keep in cache
                    vd[u][it] = __ldcs(v_rows + src);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kRows; ++u) {
            const int32_t row = row0 + u * warps;
            int32_t page, slot;
            if (row >= n_rows || !resolve_slot(table, g, seq[u], pos[u], max_blocks, error_flag, page, slot)) {
                continue;
            }
            const int64_t slot_vec = (int64_t(page) * g.page_stride_b + int64_t(slot) * g.token_stride_b) / 16;
#pragma unroll
            for (int it = 0; it < kIters; ++it) {
                const int32_t in_row = lane + 32 * it;
                if (in_row < vecs_per_row) {
                    const int32_t kvh = in_row / g.vecs_per_head_row;
                    const int32_t vec = in_row - kvh * g.vecs_per_head_row;
                    const int64_t dst = slot_vec + int64_t(kvh) * (g.head_stride_b / 16) + vec;
                    k_pool[dst] = kd[u][it];
                    v_pool[dst] = vd[u][it];
                }
            }
        }
    }
    // An unrelated plain copy riding on this launch (the host step's q rows, read from mapped host memory): four
    // vectors per thread in flight.
    const int32_t threads = int32_t(gridDim.x * blockDim.x), me = int32_t(blockIdx.x * blockDim.x + threadIdx.x);
    for (int32_t i = me; i < side_vecs; i += 4 * threads) {
        uint4 val[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (i + u * threads < side_vecs) {
                val[u] = side_src[i + u * threads];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (i + u * threads < side_vecs) {
                side_dst[i + u * threads] = val[u];
            }
        }
    }
}

// Plain copies of up to three small blocks (multiples of 16 bytes) in one launch: the host step's index arrays and q
// rows, read from mapped host memory -- a kernel's loads start sooner than a copy-engine transfer is set up.
struct CopyList {
    const uint4 *src[3];
    uint4 *dst[3];
    int32_t vecs[3];
};
__global__ void small_copies_kernel(CopyList l) {
    // lets a kernel launched behind this one with programmatic stream serialisation begin at once (it waits for these
    // copies where it needs them); no effect on an ordinary successor
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int32_t threads = int32_t(gridDim.x * blockDim.x), me = int32_t(blockIdx.x * blockDim.x + threadIdx.x);
#pragma unroll
    for (int b = 0; b < 3; ++b) {
        for (int32_t i = me; i < l.vecs[b]; i += threads) {
            l.dst[b][i] = l.src[b][i];
        }
    }
}

__global__ void paged_gather_kernel(const uint4 *__restrict__ k_pool, const uint4 *__restrict__ v_pool,
                                    uint4 *__restrict__ k_out, uint4 *__restrict__ v_out,
                                    const int32_t *__restrict__ table, CopyGeom g, int32_t seq_row, int32_t n_tokens,
                                    int32_t max_blocks, int32_t *error_flag) {
    const int32_t vecs_per_row = g.vecs_per_head_row * g.nkvh;
    const int64_t total = int64_t(n_tokens) * 2 * vecs_per_row;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int32_t tok = int32_t(i / (2 * vecs_per_row));
        const int32_t r = int32_t(i - int64_t(tok) * 2 * vecs_per_row);
        const int32_t is_v = r / vecs_per_row;
        const int32_t in_row = r - is_v * vecs_per_row;
        const int32_t kvh = in_row / g.vecs_per_head_row;
        const int32_t vec = in_row - kvh * g.vecs_per_head_row;
        int32_t page, slot;
        if (!resolve_slot(table, g, seq_row, tok, max_blocks, error_flag, page, slot)) {
            continue;
        }
        const int64_t off_b = int64_t(page) * g.page_stride_b + int64_t(kvh) * g.head_stride_b +
                              int64_t(slot) * g.token_stride_b;
        const uint4 val = (is_v ? v_pool : k_pool)[off_b / 16 + vec];
        (is_v ? v_out : k_out)[int64_t(tok) * vecs_per_row + in_row] = val;
    }
}

CopyGeom make_geom(const KVView &kv, size_t elem_size) {
    CHECK_ARGUMENT((size_t(kv.d) * elem_size) % 16 == 0, "paged copy: head rows must be a multiple of 16 bytes");
    CHECK_ARGUMENT((size_t(kv.token_stride) * elem_size) % 16 == 0 && (size_t(kv.head_stride) * elem_size) % 16 == 0 &&
                       (size_t(kv.page_stride) * elem_size) % 16 == 0,
                   "paged copy: strides must be multiples of 16 bytes");
    CopyGeom g;
    g.page_stride_b = kv.page_stride * int64_t(elem_size);
    g.head_stride_b = kv.head_stride * int64_t(elem_size);
    g.token_stride_b = kv.token_stride * int64_t(elem_size);
    g.vecs_per_head_row = int32_t(size_t(kv.d) * elem_size / 16);
    g.nkvh = kv.nkvh;
    g.page_size = kv.page_size;
    g.num_pages = kv.num_pages;
    g.table_stride = kv.table_stride;
    return g;
}

int grid_for(int64_t threads, int block) {
    const int64_t want = (threads + block - 1) / block;
    const int64_t cap = 148 * 8;
    return int(want < cap ? (want ? want : 1) : cap);
}

// K1b: the step just before attention, fused. Input is the packed projection output qkv [rows, (nh + 2 nkvh) * d] (plus
// an optional bias row); q and k heads get the half-split rotary embedding (angle = pos / theta^(2j/d) in f32, as the
// rope operator), q goes to a contiguous [rows, nh, d] tensor, k and v go straight into their page slots. One thread
// handles VEC elements of the lower half of a head row and the matching VEC of the upper half (VEC = 16 bytes of T, or
// 1 when d is not a multiple of 2 VEC): f32 arithmetic, one rounding.
template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack {
    T v[VEC];
};

template <typename T, int VEC, bool kPerHead>
__global__ void paged_rope_append_kernel(unsigned char *__restrict__ k_pool, unsigned char *__restrict__ v_pool,
                                         T *__restrict__ q_out, const T *__restrict__ qkv, const T *__restrict__ bias,
                                         const int32_t *__restrict__ table, const int32_t *__restrict__ seq_ids,
                                         const int32_t *__restrict__ positions, CopyGeom g, int32_t n_rows, int32_t nh,
                                         int32_t d, float theta, int32_t max_blocks, int32_t *error_flag) {
    using P = Pack<T, VEC>;
    // Under a programmatic launch: let the next kernel (the decode attention) start its set-up, then wait for the
    // projection that produced qkv.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    // theta^(2j/d) for the d/2 pair indices, once per CTA instead of one powf per element (before the wait: it depends
    // on nothing the previous kernel writes)
    extern __shared__ float s_divisor[];
    const int32_t half = d / 2;
    for (int32_t j = threadIdx.x; j < half; j += blockDim.x) {
        s_divisor[j] = powf(theta, 2.f * float(j) / float(d));
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // A thread owns VEC pair indices of one row and every head_groups-th head: the sines and cosines depend on
    // (position, pair index) only, so they are computed once and reused for the thread's heads. Large calls (prefill)
    // use few groups -- less transcendental work per byte; small ones (a decode step) one group per head -- the
    // shortest dependent chain per thread.
    const int32_t vec_per_head = half / VEC;
    const int32_t heads = nh + 2 * g.nkvh;
    const int32_t head_groups = kPerHead ? heads : 4; // kPerHead: one head per thread (small calls)
    const int64_t total = int64_t(n_rows) * head_groups * vec_per_head;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const int64_t row_elems = int64_t(heads) * d;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int32_t row = int32_t(i / (head_groups * vec_per_head));
        const int32_t r = int32_t(i - int64_t(row) * head_groups * vec_per_head);
        const int32_t first_head = r / vec_per_head;
        const int32_t j0 = (r - first_head * vec_per_head) * VEC;
        const int32_t pos = positions[row];
        float sn[VEC], cs[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            sincosf(float(pos) / s_divisor[j0 + e], &sn[e], &cs[e]);
        }
        int32_t page = 0, slot = 0;
        // The slot lookup (three dependent loads) is needed only by threads that reach a K or V head: a one-head thread
        // of a small call does it on demand; a many-head thread of a large call starts it up front, under its other loads.
        bool resolved = false, slot_ok = false;
        if (head_groups < heads) {
            slot_ok = resolve_slot(table, g, seq_ids[row], pos, max_blocks, error_flag, page, slot);
            resolved = true;
        }
        for (int32_t head = first_head; head < heads; head += head_groups) {
            const int64_t in_off = int64_t(row) * row_elems + int64_t(head) * d + j0;
            P lo = *reinterpret_cast<const P *>(qkv + in_off);
            P hi = *reinterpret_cast<const P *>(qkv + in_off + half);
            float a[VEC], b[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                a[e] = to_f32(lo.v[e]);
                b[e] = to_f32(hi.v[e]);
            }
            if (bias != nullptr) {
                const P blo = *reinterpret_cast<const P *>(bias + int64_t(head) * d + j0);
                const P bhi = *reinterpret_cast<const P *>(bias + int64_t(head) * d + j0 + half);
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    a[e] += to_f32(blo.v[e]);
                    b[e] += to_f32(bhi.v[e]);
                }
            }
            const bool is_v = head >= nh + g.nkvh;
            if (!is_v) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const float x = a[e], y = b[e];
                    a[e] = x * cs[e] - y * sn[e];
                    b[e] = y * cs[e] + x * sn[e];
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                lo.v[e] = from_f32<T>(a[e]);
                hi.v[e] = from_f32<T>(b[e]);
            }
            if (head < nh) {
                T *dst = q_out + (int64_t(row) * nh + head) * d + j0;
                *reinterpret_cast<P *>(dst) = lo;
                *reinterpret_cast<P *>(dst + half) = hi;
                continue;
            }
            if (!resolved) {
                slot_ok = resolve_slot(table, g, seq_ids[row], pos, max_blocks, error_flag, page, slot);
                resolved = true;
            }
            if (!slot_ok) {
                continue;
            }
            const int32_t kvh = is_v ? head - nh - g.nkvh : head - nh;
            const int64_t off_b = int64_t(page) * g.page_stride_b + int64_t(kvh) * g.head_stride_b +
                                  int64_t(slot) * g.token_stride_b + int64_t(j0) * int64_t(sizeof(T));
            unsigned char *dst = (is_v ? v_pool : k_pool) + off_b;
            *reinterpret_cast<P *>(dst) = lo;
            *reinterpret_cast<P *>(dst + int64_t(half) * int64_t(sizeof(T))) = hi;
        }
    }
}

template <typename T>
void launch_rope_append(cudaStream_t s, const KVView &kv, void *q_out, const void *qkv, const void *bias,
                        const int32_t *seq_ids, const int32_t *positions, int32_t n_rows, int32_t nh, float theta,
                        int32_t max_blocks, int32_t *error_flag) {
    constexpr int kVec = 16 / int(sizeof(T));
    const CopyGeom g = make_geom(kv, sizeof(T));
    const int32_t d = kv.d;
    auto aligned = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool wide = d % (2 * kVec) == 0 && aligned(q_out) && aligned(qkv) && aligned(bias) && aligned(kv.k_base) &&
                      aligned(kv.v_base);
    const bool per_head = n_rows <= 1024;
    const int32_t head_groups = per_head ? nh + 2 * kv.nkvh : 4;
    const int64_t threads = int64_t(n_rows) * head_groups * (d / 2 / (wide ? kVec : 1));
    const int block = 256, grid = grid_for(threads, block);
    auto *kp = static_cast<unsigned char *>(kv.k_base);
    auto *vp = static_cast<unsigned char *>(kv.v_base);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(unsigned(block));
    cfg.dynamicSmemBytes = size_t(d / 2) * sizeof(float);
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = kv.overlap_launch ? 1 : 0;
    T *qo = static_cast<T *>(q_out);
    const T *qi = static_cast<const T *>(qkv), *bi = static_cast<const T *>(bias);
    const int32_t *table = kv.block_table;
    auto go = [&](auto kernel) {
        LLAISYS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, kp, vp, qo, qi, bi, table, seq_ids, positions, g, n_rows, nh, d,
                                              theta, max_blocks, error_flag));
    };
    if (wide) {
        per_head ? go(paged_rope_append_kernel<T, kVec, true>) : go(paged_rope_append_kernel<T, kVec, false>);
    } else {
        per_head ? go(paged_rope_append_kernel<T, 1, true>) : go(paged_rope_append_kernel<T, 1, false>);
    }
}

} // namespace

void paged_append(stream_t stream, size_t elem_size, const KVView &kv, const void *k_rows, const void *v_rows,
                  const int32_t *seq_ids, const int32_t *positions, int32_t n_rows, int32_t max_blocks,
                  int32_t *error_flag, const void *side_src, void *side_dst, size_t side_bytes) {
    if (n_rows <= 0) {
        return;
    }
    CHECK_ARGUMENT(side_bytes % 16 == 0 && side_bytes / 16 < size_t(INT32_MAX), "paged append: side copy size");
    const CopyGeom g = make_geom(kv, elem_size);
    const int32_t vecs_per_row = g.vecs_per_head_row * g.nkvh;
    CHECK_ARGUMENT(vecs_per_row <= 256, "paged append: a K row of more than 4 KiB is not supported");
    const int block = 256;
    // a warp per row while that fills the GPU; from there on 2, then 4 rows per warp and pass
    const int64_t full = int64_t(148) * 8 * (block / 32);
    const int rows_per_warp = n_rows >= 4 * full ? 4 : (n_rows >= 2 * full ? 2 : 1);
    const int grid = grid_for(std::max<int64_t>(int64_t(n_rows + rows_per_warp - 1) / rows_per_warp * 32, int64_t(side_bytes / 64)), block);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(unsigned(block));
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = kv.overlap_launch ? 1 : 0;
    auto go = [&](auto kernel) {
        LLAISYS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, static_cast<uint4 *>(kv.k_base), static_cast<uint4 *>(kv.v_base),
                                              static_cast<const uint4 *>(k_rows), static_cast<const uint4 *>(v_rows),
                                              kv.block_table, seq_ids, positions, g, n_rows, max_blocks, error_flag,
                                              static_cast<const uint4 *>(side_src), static_cast<uint4 *>(side_dst),
                                              int32_t(side_bytes / 16)));
    };
    if (vecs_per_row <= 32) {
        rows_per_warp == 4 ? go(paged_append_kernel<4, 1>) : rows_per_warp == 2 ? go(paged_append_kernel<2, 1>)
                                                                               : go(paged_append_kernel<1, 1>);
    } else if (vecs_per_row <= 64) {
        rows_per_warp >= 2 ? go(paged_append_kernel<2, 2>) : go(paged_append_kernel<1, 2>);
    } else {
        go(paged_append_kernel<1, 8>);
    }
    check_launch("paged_append");
}

void small_copies(stream_t stream, const void *const *src, void *const *dst, const size_t *bytes, int n) {
    CHECK_ARGUMENT(n >= 0 && n <= 3, "small_copies: at most three blocks");
    CopyList l{};
    size_t most = 0;
    for (int i = 0; i < n; ++i) {
        CHECK_ARGUMENT(bytes[i] % 16 == 0 && bytes[i] / 16 < size_t(INT32_MAX) &&
                           reinterpret_cast<uintptr_t>(src[i]) % 16 == 0 && reinterpret_cast<uintptr_t>(dst[i]) % 16 == 0,
                       "small_copies: blocks must be 16-byte aligned multiples of 16 bytes");
        l.src[i] = static_cast<const uint4 *>(src[i]);
        l.dst[i] = static_cast<uint4 *>(dst[i]);
        l.vecs[i] = int32_t(bytes[i] / 16);
        most = std::max(most, bytes[i] / 16);
    }
    if (most == 0) {
        return;
    }
    const int block = 256;
    small_copies_kernel<<<grid_for(int64_t(most), block), block, 0, static_cast<cudaStream_t>(stream)>>>(l);
    check_launch("small_copies");
}

void paged_gather(stream_t stream, size_t elem_size, const KVView &kv, int32_t seq_row, int32_t n_tokens,
                  void *k_out, void *v_out, int32_t *error_flag) {
    if (n_tokens <= 0) {
        return;
    }
    const CopyGeom g = make_geom(kv, elem_size);
    const int block = 256;
    const int grid = grid_for(int64_t(n_tokens) * 2 * g.vecs_per_head_row * g.nkvh, block);
    paged_gather_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(kv.k_base), static_cast<const uint4 *>(kv.v_base), static_cast<uint4 *>(k_out),
        static_cast<uint4 *>(v_out), kv.block_table, g, seq_row, n_tokens,
        kv.block_table ? kv.table_stride : INT32_MAX, error_flag);
    check_launch("paged_gather");
}

void paged_rope_append(stream_t stream, llaisysDataType_t dtype, const KVView &kv, void *q_out, const void *qkv,
                       const void *bias, const int32_t *seq_ids, const int32_t *positions, int32_t n_rows, int32_t nh,
                       float theta, int32_t max_blocks, int32_t *error_flag) {
    if (n_rows <= 0) {
        return;
    }
    CHECK_ARGUMENT(kv.d % 2 == 0, "rope append: head_dim must be even");
    auto s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        launch_rope_append<float>(s, kv, q_out, qkv, bias, seq_ids, positions, n_rows, nh, theta, max_blocks, error_flag);
        break;
    case LLAISYS_DTYPE_F16:
        launch_rope_append<__half>(s, kv, q_out, qkv, bias, seq_ids, positions, n_rows, nh, theta, max_blocks, error_flag);
        break;
    case LLAISYS_DTYPE_BF16:
        launch_rope_append<__nv_bfloat16>(s, kv, q_out, qkv, bias, seq_ids, positions, n_rows, nh, theta, max_blocks,
                                          error_flag);
        break;
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
    check_launch("paged_rope_append");
}

} // namespace llaisys::kernels
