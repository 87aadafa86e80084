// K6: weight-streaming projection for a decode step, out[M, N] (+)= x[M, K] . W[N, K]^T with M <= 128 rows, on the
// 5th-generation tensor cores (tcgen05 + TMEM), operands staged by TMA.
//
// Roofline: HBM. With at most 128 activation rows every weight is used once per step: algorithmic bytes per launch =
// N * K * 2 (the weights) + M * K * 2 + M * N * 2 (activations in and out). The arithmetic (2 M N K flops) is a few
// per cent of the tensor pipe; the kernel's job is to keep enough weight bytes in flight.
//
// One CTA per (tile of 128 output features, K split). The WEIGHT tile is the A operand (128 TMEM lanes = output
// features) and the activations are the B operand (MMA N = rows rounded up to 32), so a stage moves 16 KiB of weights
// for at most 16 KiB of activations (which come from L2) and nothing is padded to the tensor core's 128-row side. Both
// operands are K-major with the 128-byte swizzle, 64 K-elements per pipeline stage:
//   thread 0   (producer) issues the TMA loads of a stage: the weight tile first -- weights do not depend on the
//              previous kernel, so under a programmatic launch the first stages are already in flight when the
//              previous kernel finishes -- then the activation tile;
//   thread 32  (MMA) issues four tcgen05.mma (M 128, N rows, K 16) per stage and commits the stage's "empty" barrier;
//   all 128    threads run the epilogue from TMEM: thread = output feature, TMEM columns = rows of the activation.
// Projections with few feature tiles (N = 1536 gives 12) split K over a thread-block cluster of up to 8 CTAs: each CTA
// parks its f32 partial tile in its own shared memory, and after a cluster barrier CTA r sums rows r, r + S, ... of all
// S partials through distributed shared memory in rank order (deterministic) and stores them. No global scratch, no
// atomics, no multicast.
//
// Every mbarrier wait is bounded; a wait that runs out sets the error word and the CTA skips its stores but still
// takes part in both cluster barriers and frees its TMEM.
#include "kernels.hpp"
#include "tcgen05_utils.cuh"

#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

namespace llaisys::kernels {

namespace {

constexpr int kBF = 128;                // output features per tile = TMEM lanes
constexpr int kBK = 64;                 // K elements per stage: one 128-byte swizzled row
constexpr int kThreads = 128;
constexpr int kWStageBytes = kBF * 128; // 16 KiB
constexpr int kMaxStages = 10;
constexpr int kMaxSplit = 8;            // portable cluster size
constexpr int kRingBudget = 196 * 1024; // bytes of shared memory given to the stage ring
constexpr int kErrGemmTimeout = 16;
constexpr int kNumBars = 2 * kMaxStages + 1;

struct GemmParams {
    void *out;
    int32_t m, n, k;
    int32_t rows_pad; // m rounded up to 32: the MMA's N and the activation box height
    int32_t stages;
    int32_t accumulate;
    int32_t *error_flag;
};

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// 16 bytes of a peer CTA's shared memory (same offset as local_addr in this CTA). Not volatile: the loads of a
// reduction are independent and may be issued back to back; the cluster barrier before them orders them.
__device__ __forceinline__ float4 ld_peer_f4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_addr), "r"(rank));
    float4 v;
    asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
    return v;
}

template <bool kBf16>
__device__ __forceinline__ float unpack_lo(uint32_t w) {
    if constexpr (kBf16) {
        return __uint_as_float(w << 16);
    } else {
        return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu)));
    }
}
template <bool kBf16>
__device__ __forceinline__ float unpack_hi(uint32_t w) {
    if constexpr (kBf16) {
        return __uint_as_float(w & 0xffff0000u);
    } else {
        return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
    }
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
    skinny_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t base_u32 = (raw_u32 + 1023u) & ~1023u;
    unsigned char *base = smem_raw + (base_u32 - raw_u32);
    const int stage_bytes = kWStageBytes + p.rows_pad * 128;
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + p.stages * stage_bytes);
    const uint32_t bars_u32 = smem_u32(bars);
    uint32_t *s_tmem_base = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem_base + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tile = blockIdx.x;
    const int n_split = gridDim.y;
    const int split = blockIdx.y;
    const int chunks = p.k / kBK;
    const int c0 = int((long long)split * chunks / n_split), c1 = int((long long)(split + 1) * chunks / n_split);
    const int n_chunks = c1 - c0;
    const uint32_t tmem_cols = p.rows_pad <= 32 ? 32u : (p.rows_pad <= 64 ? 64u : 128u);

    auto full_bar = [&](int st) { return bars_u32 + uint32_t(st) * 8; };
    auto empty_bar = [&](int st) { return bars_u32 + uint32_t(kMaxStages + st) * 8; };
    const uint32_t accum_bar = bars_u32 + uint32_t(2 * kMaxStages) * 8;
    auto w_stage = [&](int st) { return base_u32 + uint32_t(st * stage_bytes); };
    auto x_stage = [&](int st) { return base_u32 + uint32_t(st * stage_bytes + kWStageBytes); };

    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            mbar_init(bars_u32 + i * 8, 1);
        }
        *s_abort = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(s_tmem_base), tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;
    grid_launch_dependents();

    auto give_up = [&]() {
        *s_abort = 1;
        atomicOr(p.error_flag, kErrGemmTimeout);
    };

    if (tid == 0) {
        // ================================ producer ================================
        // Weight tiles of the first ring-full of stages go out before the wait on the previous kernel.
        const int head = n_chunks < p.stages ? n_chunks : p.stages;
        for (int i = 0; i < head; ++i) {
            mbar_arrive_expect_tx(full_bar(i), uint32_t(stage_bytes));
            tma_load_2d(w_stage(i), &tmap_w, (c0 + i) * kBK, n_tile * kBF, full_bar(i));
        }
        grid_dependency_wait();
        for (int i = 0; i < head; ++i) {
            tma_load_2d(x_stage(i), &tmap_x, (c0 + i) * kBK, 0, full_bar(i));
        }
        for (int i = head; i < n_chunks; ++i) {
            const int st = i % p.stages;
            if (!wait_or_abort(empty_bar(st), uint32_t(i / p.stages - 1) & 1u, s_abort)) {
                give_up();
                break;
            }
            mbar_arrive_expect_tx(full_bar(st), uint32_t(stage_bytes));
            tma_load_2d(w_stage(st), &tmap_w, (c0 + i) * kBK, n_tile * kBF, full_bar(st));
            tma_load_2d(x_stage(st), &tmap_x, (c0 + i) * kBK, 0, full_bar(st));
        }
    } else if (tid == 32) {
        // ================================ MMA issue ================================
        const uint32_t idesc = make_idesc(kBf16, false, kBF, p.rows_pad);
        bool ok = true;
        for (int i = 0; i < n_chunks && ok; ++i) {
            const int st = i % p.stages;
            ok = wait_or_abort(full_bar(st), uint32_t(i / p.stages) & 1u, s_abort);
            if (!ok) {
                break;
            }
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < kBK / 16; ++ks) {
                const uint64_t a = smem_desc_sw128(w_stage(st) + ks * 32, 0, 1024);
                const uint64_t b = smem_desc_sw128(x_stage(st) + ks * 32, 0, 1024);
                umma_f16(tmem_base, a, b, idesc, (i > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit(empty_bar(st));
        }
        if (ok) {
            umma_commit(accum_bar);
        } else {
            give_up();
        }
    }
    __syncwarp();
    // The accumulate path reads `out`, which the previous kernel may have written: every thread orders itself after it.
    grid_dependency_wait();

    // ================================ epilogue ================================
    const bool done = wait_or_abort(accum_bar, 0u, s_abort);
    if (!done && tid == 0) {
        give_up();
    }
    tc_fence_after();
    const int f_local = warp * 32 + lane;                  // TMEM lane = output feature inside the tile
    const long long f = (long long)n_tile * kBF + f_local; // output column
    const uint32_t taddr = tmem_base + (uint32_t(warp * 32) << 16);
    {
        // The ring is idle now (every load was consumed, every MMA has completed): park the f32 tile in it as
        // [row][128 features] -- a warp's 32 features of one row are 128 contiguous bytes -- so that the stores below are
        // 8-byte pieces of contiguous output rows whatever the split.
        const uint32_t part_u32 = base_u32;
        for (int c = 0; c < p.rows_pad / 32; ++c) {
            float v[32];
            tmem_ld32(taddr + c * 32, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(part_u32 + uint32_t((c * 32 + j) * kBF + f_local) * 4), "f"(v[j])
                             : "memory");
            }
        }
        if (n_split > 1) {
            __syncwarp();
            cluster_arrive();
            cluster_wait();
        } else {
            __syncthreads();
        }
        // CTA r of the cluster finishes rows r, r + S, r + 2S, ... (< M). A thread owns 4 consecutive features of a row:
        // one 16-byte read per peer (all issued before the first add), the S partials added in rank order.
        const int rank = n_split > 1 ? int(cluster_rank()) : 0;
        const int my_rows = p.m > rank ? (p.m - rank + n_split - 1) / n_split : 0;
        for (int idx = tid; idx < my_rows * (kBF / 4); idx += kThreads) {
            const int t = rank + (idx / (kBF / 4)) * n_split;
            const int f4 = (idx % (kBF / 4)) * 4;
            const uint32_t local = part_u32 + uint32_t(t * kBF + f4) * 4;
            const long long o = (long long)t * p.n + (long long)n_tile * kBF + f4;
            uint2 *dst = reinterpret_cast<uint2 *>(static_cast<unsigned char *>(p.out) + o * 2);
            uint2 old = make_uint2(0u, 0u);
            if (p.accumulate) {
                old = *dst;
            }
            float4 acc;
            if (n_split > 1) {
                float4 part[kMaxSplit];
#pragma unroll
                for (int peer = 0; peer < kMaxSplit; ++peer) {
                    if (peer < n_split) {
                        part[peer] = ld_peer_f4(local, uint32_t(peer));
                    }
                }
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int peer = 0; peer < kMaxSplit; ++peer) {
                    if (peer < n_split) {
                        acc.x += part[peer].x;
                        acc.y += part[peer].y;
                        acc.z += part[peer].z;
                        acc.w += part[peer].w;
                    }
                }
            } else {
                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                             : "=f"(acc.x), "=f"(acc.y), "=f"(acc.z), "=f"(acc.w)
                             : "r"(local)
                             : "memory");
            }
            if (p.accumulate) {
                acc.x += unpack_lo<kBf16>(old.x);
                acc.y += unpack_hi<kBf16>(old.x);
                acc.z += unpack_lo<kBf16>(old.y);
                acc.w += unpack_hi<kBf16>(old.y);
            }
            if (done) {
                *dst = make_uint2(pack2<kBf16>(acc.x, acc.y), pack2<kBf16>(acc.z, acc.w));
            }
        }
        if (n_split > 1) {
            __syncwarp();
            cluster_arrive(); // no CTA leaves while a peer may still read its partial tile
            cluster_wait();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn gemm_encode_fn() {
    static EncodeTiledFn fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) != cudaSuccess ||
            res != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            return EncodeTiledFn(nullptr);
        }
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// Row-major [rows, k] 16-bit matrix -> 2-D map with a box of 64 elements x box_rows rows, 128-byte swizzle. Maps are
// cached: a decode loop asks for the same handful of (pointer, shape) pairs every step.
bool matrix_map(CUtensorMap *out, const void *ptr, uint64_t rows, uint64_t k, uint32_t box_rows, bool bf16) {
    using Key = std::tuple<const void *, uint64_t, uint64_t, uint32_t, bool, int>;
    static std::mutex mu;
    static std::map<Key, CUtensorMap> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        return false;
    }
    const Key key{ptr, rows, k, box_rows, bf16, dev};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn encode = gemm_encode_fn();
    if (encode == nullptr) {
        return false;
    }
    const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(k * 2)};
    const cuuint32_t box[2] = {cuuint32_t(kBK), box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    CUtensorMap map;
    const CUresult rc = encode(&map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                               const_cast<void *>(ptr), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        return false;
    }
    if (cache.size() > 4096) {
        cache.clear(); // callers with ever-changing buffers: start over rather than grow without bound
    }
    cache.emplace(key, map);
    *out = map;
    return true;
}

int32_t *gemm_error_word() {
    static std::mutex mu;
    static std::map<int, int32_t *> words;
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    auto it = words.find(dev);
    if (it != words.end()) {
        return it->second;
    }
    int32_t *w = nullptr;
    LLAISYS_CUDA_CHECK(cudaMalloc(&w, sizeof(int32_t)));
    LLAISYS_CUDA_CHECK(cudaMemset(w, 0, sizeof(int32_t)));
    words.emplace(dev, w);
    return w;
}

template <bool kBf16>
void launch_gemm(cudaStream_t s, const CUtensorMap &tx, const CUtensorMap &tw, const GemmParams &p, int tiles, int split,
                 size_t smem_bytes, bool overlap) {
    static std::once_flag once[64];
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    std::call_once(once[dev & 63], [] {
        LLAISYS_CUDA_CHECK(cudaFuncSetAttribute(skinny_gemm_tc_kernel<kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                int(1024 + kRingBudget + kNumBars * 8 + 16)));
    });
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(tiles), unsigned(split), 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attrs[2];
    int n_attrs = 0;
    if (split > 1) {
        attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
        attrs[n_attrs].val.clusterDim.x = 1;
        attrs[n_attrs].val.clusterDim.y = unsigned(split);
        attrs[n_attrs].val.clusterDim.z = 1;
        ++n_attrs;
    }
    if (overlap) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = unsigned(n_attrs);
    LLAISYS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, skinny_gemm_tc_kernel<kBf16>, tx, tw, p));
}

} // namespace

bool linear_tc(stream_t stream, llaisysDataType_t dtype, void *out, const void *in, const void *weight, size_t m, size_t n,
               size_t k, bool accumulate, bool overlap) {
    const bool bf16 = dtype == LLAISYS_DTYPE_BF16;
    auto aligned = [](const void *ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    if (!(bf16 || dtype == LLAISYS_DTYPE_F16) || m == 0 || m > 128 || k == 0 || k % kBK != 0 || n == 0 || n % kBF != 0 ||
        !aligned(out) || !aligned(in) || !aligned(weight) || n > (size_t(1) << 30) || k > (size_t(1) << 30)) {
        return false;
    }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        (void)cudaGetLastError();
        return false;
    }
    const int tiles = int(n / size_t(kBF));
    if (tiles > 2 * sms) {
        return false; // vocabulary-sized projections: many waves of one-tile CTAs lose to a persistent library kernel
    }
    // few feature tiles: split K over a cluster until the grid fills the GPU
    const int chunks = int(k / kBK);
    int split = sms / tiles;
    split = split < 1 ? 1 : (split > kMaxSplit ? kMaxSplit : split);
    split = split > chunks ? chunks : split;
    GemmParams p;
    p.out = out;
    p.m = int32_t(m);
    p.n = int32_t(n);
    p.k = int32_t(k);
    p.rows_pad = int32_t((m + 31) / 32 * 32);
    const int stage_bytes = kWStageBytes + p.rows_pad * 128;
    int stages = kRingBudget / stage_bytes;
    stages = stages > kMaxStages ? kMaxStages : stages;
    p.stages = stages;
    p.accumulate = accumulate ? 1 : 0;
    p.error_flag = gemm_error_word();
    CUtensorMap tx, tw;
    if (!matrix_map(&tx, in, m, k, uint32_t(p.rows_pad), bf16) || !matrix_map(&tw, weight, n, k, uint32_t(kBF), bf16)) {
        return false;
    }
    const size_t smem_bytes = 1024 + size_t(stages) * stage_bytes + kNumBars * 8 + 16;
    auto s = static_cast<cudaStream_t>(stream);
    if (bf16) {
        launch_gemm<true>(s, tx, tw, p, tiles, split, smem_bytes, overlap);
    } else {
        launch_gemm<false>(s, tx, tw, p, tiles, split, smem_bytes, overlap);
    }
    check_launch("skinny_gemm_tc");
    return true;
}

int linear_tc_status(stream_t stream) {
    int32_t *w = gemm_error_word();
    int32_t host = 0;
    auto s = static_cast<cudaStream_t>(stream);
    LLAISYS_CUDA_CHECK(cudaMemcpyAsync(&host, w, sizeof(host), cudaMemcpyDeviceToHost, s));
    LLAISYS_CUDA_CHECK(cudaStreamSynchronize(s));
    if (host != 0) {
        LLAISYS_CUDA_CHECK(cudaMemsetAsync(w, 0, sizeof(host), s));
    }
    return host;
}

} // namespace llaisys::kernels
