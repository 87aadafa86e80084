// K2 + K3: split-KV flash decoding over a paged (or contiguous) 16-bit K/V view, head_dim 128, page 16,
// one query token per sequence, GQA group <= 8 -- with the log-sum-exp combine fused in.
//
// Roofline: HBM. Algorithmic bytes per launch = sum_s ctx_s * (2 * nkvh * 128 * 2)   K and V read once
//                                             + 2 * n_seqs * nh * 128 * 2            q read, out written
//                                             + 4 * sum_s ceil(ctx_s / 16)           block-table entries
// i.e. 1024 B per cached token for 2 kv heads. Every K/V byte is fetched from HBM once and used by all
// query heads of its GQA group.
//
// Work decomposition ("even page split"): the pages of all (sequence, kv-head) pairs are laid end to end,
//     pair p = (s, kvh) occupies [cum[s] * nkvh + kvh * np(s), ... + np(s)),   np(s) = ceil(ctx_s / 16),
// and the launch's G persistent CTAs (two per SM) each take one contiguous span of ceil(T / G) pages. Ragged
// context lengths therefore cost nothing in balance, there is no tail wave, and the copy pipeline of a CTA
// keeps streaming across pair boundaries. A pair that is cut by span boundaries is finished by whichever of
// its CTAs arrives last (one atomic counter per pair, no waiting): at most G + n_pairs partial results exist,
// a few hundred KB against hundreds of MB of K/V.
//
// Inside a CTA (4 warps): K/V tiles (16 tokens x 128 dims x 2 B = 4 KiB) are copied global -> shared with
// 16-byte cp.async into a 3-stage ring of 4 pages (32 KiB per stage), XOR-swizzled on the 16-byte chunk index
// so that ldmatrix reads are bank-conflict free. Warp w owns page w of each stage and keeps its own running
// (max, sum, O) -- merged across warps only when a pair ends. The arithmetic runs on the warp-level tensor
// cores (mma.sync m16n8k16, f32 accumulate) with the K/V tile as the 16-row operand and the query heads of the
// group, padded to 8, as the 8-column operand:
//     S^T[16 tok x 8 heads] = K[16 x 128] . Q^T[128 x 8]           8 MMAs
//     O^T[128 x 8 heads]   += V^T[128 x 16 tok] . P[16 tok x 8]    8 MMAs (P moved C-fragment -> B-fragment
//                                                                   with movmatrix, V^T read with ldmatrix.trans)
// so one K/V byte costs ~1/256 of an MMA and the CUDA cores only do the 4-values-per-thread softmax.
// (tcgen05 is kept for the prefill kernel's dense tiles; a decode step has 6 query rows per K/V tile, far
// below a 128-row UMMA tile.)
//
// Rows past a sequence's length inside its last page are zero-filled by the copy (src-size 0), never read
// from the pool; out-of-range block-table entries are skipped and flagged in the error word.
#include "kernels.hpp"

#include <cmath>
#include "decode_epilogue.cuh"
#include "mma_utils.cuh"

#include <mutex>

namespace llaisys::kernels {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kPagesPerStage = kWarps; // one page per warp per stage
constexpr int kStages = 3;
constexpr int kPage = 16;
constexpr int kD = 128;
constexpr int kTileBytes = kPage * kD * 2;            // one (page, K or V, kv-head) tile
constexpr int kPageBytes = 2 * kTileBytes;            // K tile followed by V tile
constexpr int kStageBytes = kPagesPerStage * kPageBytes;
constexpr int kRingBytes = kStages * kStageBytes;     // 96 KiB
constexpr int kMaxGroup = 8;
constexpr int kMaxSeqs = 1024;                        // prefix sums of page counts live in shared memory
constexpr int kCtasPerSm = 2;
static_assert(kThreads == kD, "the pair epilogue maps one thread to one output dimension");

struct DecodeParams {
    const char *k_base;
    const char *v_base;
    long long page_stride_b, head_stride_b, token_stride_b;
    const int32_t *block_table; // null: block b is page b
    int32_t table_stride, num_pages, max_tokens;
    const int32_t *seq_ids; // null: row s
    const int32_t *kv_lens; // null: const_kv_len
    int32_t const_kv_len;
    int32_t n_seqs, nkvh, group, nh;
    const void *q;  // [n_seqs, nh, 128]
    void *out;      // [n_seqs, nh, 128] or null
    float *part;    // [n_seqs, nh, 130] or null
    float scale_log2;
    float *partials;   // [gridDim.x + n_pairs][group][130]
    int32_t *counters; // [n_pairs], zero on entry and on exit
    int32_t *error_flag;
};

// ---- walking a span of the flattened page list -----------------------------------------------------

struct Cursor {
    int s, kvh, j, np, kv_len, remaining; // sequence, kv-head, next local page, pages of s, tokens of s, pages left
};

struct Stage {
    int s, kvh, j, n, kv_len; // n pages [j, j + n) of pair (s, kvh)
    bool seg_end;             // last stage of this pair inside the CTA's span
};

__device__ __forceinline__ int seq_kv_len(const DecodeParams &p, int s) {
    int len = p.kv_lens ? p.kv_lens[s] : p.const_kv_len;
    return min(max(len, 0), p.max_tokens);
}

// Hands out the next (at most kPagesPerStage) pages of the span; never crosses a pair boundary.
__device__ __forceinline__ Stage cursor_next(Cursor &c, const int *cum, const DecodeParams &p) {
    Stage st;
    st.s = c.s;
    st.kvh = c.kvh;
    st.j = c.j;
    st.kv_len = c.kv_len;
    st.n = min(kPagesPerStage, min(c.np - c.j, c.remaining));
    c.j += st.n;
    c.remaining -= st.n;
    st.seg_end = (c.j == c.np) || (c.remaining == 0);
    if (c.j == c.np && c.remaining > 0) {
        c.j = 0;
        if (++c.kvh == p.nkvh) {
            c.kvh = 0;
            do { // remaining > 0 guarantees a later sequence with pages; the bound only guards the walk
                ++c.s;
                c.np = cum[c.s + 1] - cum[c.s];
            } while (c.np == 0 && c.s + 1 < p.n_seqs);
            c.kv_len = seq_kv_len(p, c.s);
        }
    }
    return st;
}

// ---- the kernel -----------------------------------------------------------------------------------

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) paged_decode_split_kernel(DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char *ring = smem_raw;                                               // kRingBytes
    float *red_o = reinterpret_cast<float *>(smem_raw + kRingBytes);              // [kWarps][group][kD]
    float *red_ml = red_o + kWarps * p.group * kD;                                // [kWarps][kMaxGroup][2]
    int *cum = reinterpret_cast<int *>(red_ml + kWarps * kMaxGroup * 2);          // [n_seqs + 1]
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, q4 = lane & 3; // MMA fragment coordinates: row group, column pair

    // -- prefix sums of page counts (warp 0), then the span of this CTA ---------------------------------
    if (warp == 0) {
        int running = 0;
        if (lane == 0) {
            cum[0] = 0;
        }
        for (int base = 0; base < p.n_seqs; base += 32) {
            const int s = base + lane;
            int np = 0;
            if (s < p.n_seqs) {
                np = (seq_kv_len(p, s) + kPage - 1) / kPage;
            }
            int incl = np;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) {
                    incl += up;
                }
            }
            if (s < p.n_seqs) {
                cum[s + 1] = running + incl;
            }
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();

    const int n_pairs = p.n_seqs * p.nkvh;
    const long long total = (long long)cum[p.n_seqs] * p.nkvh;
    const int span = int((total + gridDim.x - 1) / gridDim.x);
    const long long x0 = (long long)blockIdx.x * span;
    const long long x1 = min(total, x0 + span);

    // -- sequences without any token: the output row is zero (partial: o = 0, m = -inf, l = 0) ----------
    for (int pair = blockIdx.x; pair < n_pairs; pair += gridDim.x) {
        const int s = pair / p.nkvh, kvh = pair - s * p.nkvh;
        if (cum[s + 1] - cum[s] != 0) {
            continue;
        }
        for (int h = 0; h < p.group; ++h) {
            const long long row = (long long)s * p.nh + kvh * p.group + h;
            if (p.part != nullptr) {
                p.part[row * (kD + 2) + tid] = 0.f;
                if (tid == 0) {
                    p.part[row * (kD + 2) + kD] = -INFINITY;
                    p.part[row * (kD + 2) + kD + 1] = 0.f;
                }
            } else {
                store_out<kBf16>(p.out, row * kD + tid, 0.f);
            }
        }
    }
    if (x0 >= x1) {
        return;
    }

    // -- locate the first page of the span ---------------------------------------------------------------
    Cursor load_c;
    {
        int lo = 0, hi = p.n_seqs - 1;
        while (lo < hi) { // last s with cum[s] * nkvh <= x0
            const int mid = (lo + hi + 1) >> 1;
            if ((long long)cum[mid] * p.nkvh <= x0) {
                lo = mid;
            } else {
                hi = mid - 1;
            }
        }
        // cum is non-decreasing and x0 < total, so the last s with cum[s] * nkvh <= x0 also has
        // x0 < cum[s + 1] * nkvh: it owns page x0 and is never an empty sequence.
        load_c.s = lo;
        load_c.np = cum[lo + 1] - cum[lo];
        const int r = int(x0 - (long long)cum[lo] * p.nkvh);
        load_c.kvh = r / load_c.np;
        load_c.j = r - load_c.kvh * load_c.np;
        load_c.kv_len = seq_kv_len(p, lo);
        load_c.remaining = int(x1 - x0);
    }
    Cursor comp_c = load_c;

    const uint32_t ring_u32 = smem_u32(ring);

    // Copies one stage: iteration `it` moves half a tile -- (page it/4, K or V, tokens (it&1)*8 .. +8) -- with every
    // thread carrying 16 bytes, so global reads are fully coalesced 2 KiB runs.
    auto issue_stage = [&](const Stage &st, int slot) {
        const int seq_row = p.seq_ids ? p.seq_ids[st.s] : st.s;
        const uint32_t stage_base = ring_u32 + slot * kStageBytes;
        const int cc = tid & 15;
#pragma unroll
        for (int pg = 0; pg < kPagesPerStage; ++pg) {
            if (pg >= st.n) {
                break;
            }
            const int blk = st.j + pg;
            int page = blk;
            if (p.block_table != nullptr) {
                page = p.block_table[(long long)seq_row * p.table_stride + blk];
            }
            bool page_ok = page >= 0 && page < p.num_pages;
            if (!page_ok) {
                if (tid == 0) {
                    atomicOr(p.error_flag, kErrBadPage);
                }
                page = 0;
            }
            const long long page_off = (long long)page * p.page_stride_b + (long long)st.kvh * p.head_stride_b;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int tok = half * 8 + (tid >> 4);
                const bool valid = page_ok && (blk * kPage + tok < st.kv_len);
                const long long off = page_off + (long long)tok * p.token_stride_b + cc * 16;
                const uint32_t dst = stage_base + pg * kPageBytes + tok * (kD * 2) + ((cc ^ (tok & 7)) << 4);
                cp_async_16(dst, p.k_base + (valid ? off : 0), valid ? 16 : 0);
                cp_async_16(dst + kTileBytes, p.v_base + (valid ? off : 0), valid ? 16 : 0);
            }
        }
    };

    // -- prologue: fill kStages - 1 stages ----------------------------------------------------------------
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        if (load_c.remaining > 0) {
            const Stage st = cursor_next(load_c, cum, p);
            issue_stage(st, i);
        }
        cp_async_commit();
    }

    // -- per-warp running state for the current pair ----------------------------------------------------
    float m2[2], l[2], o_acc[8][4];
    uint32_t qf[8][2];
    bool new_pair = true;
    auto reset_state = [&]() {
        m2[0] = m2[1] = -INFINITY;
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            o_acc[mt][0] = o_acc[mt][1] = o_acc[mt][2] = o_acc[mt][3] = 0.f;
        }
    };
    reset_state();

    // per-lane constant parts of the ldmatrix addresses (see the fragment maps in the header comment)
    const int lm_r = lane & 7, lm_mi = lane >> 3;
    const int k_tok = lm_r + 8 * (lm_mi & 1), k_cc0 = lm_mi >> 1; // K tile, non-transposed: chunk = 2 * ks + k_cc0
    const int v_tok = lm_r + 8 * (lm_mi >> 1), v_cc0 = lm_mi & 1; // V tile, transposed:     chunk = 2 * mt + v_cc0

    int it = 0;
    while (comp_c.remaining > 0) {
        cp_async_wait<kStages - 2>();
        __syncthreads(); // stage `it` has landed for every thread, and everyone is done with stage it - 1
        if (load_c.remaining > 0) {
            const Stage st = cursor_next(load_c, cum, p);
            issue_stage(st, (it + kStages - 1) % kStages);
        }
        cp_async_commit();

        const Stage st = cursor_next(comp_c, cum, p);
        if (st.n <= 0) { // cannot happen with consistent lengths; leave rather than spin (uniform over the CTA)
            if (tid == 0) {
                atomicOr(p.error_flag, kErrBadSeq);
            }
            break;
        }
        if (new_pair) {
            // query fragments of this pair: B operand [k = dim][n = head], head g of the group (zero beyond it)
            const uint32_t *q_row = reinterpret_cast<const uint32_t *>(
                static_cast<const char *>(p.q) + ((long long)st.s * p.nh + st.kvh * p.group + g) * (kD * 2));
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qf[ks][0] = g < p.group ? q_row[ks * 8 + q4] : 0u;
                qf[ks][1] = g < p.group ? q_row[ks * 8 + 4 + q4] : 0u;
            }
            new_pair = false;
        }

        if (warp < st.n) {
            const uint32_t tile = ring_u32 + (it % kStages) * kStageBytes + warp * kPageBytes;
            const int n_valid = min(kPage, st.kv_len - (st.j + warp) * kPage);
            // S^T = K . Q^T
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t k_row = tile + k_tok * (kD * 2);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, k_row + (((2 * ks + k_cc0) ^ lm_r) << 4));
                mma_16816<kBf16>(sc, a, qf[ks][0], qf[ks][1]);
            }
            // online softmax in the log2 domain; this thread holds tokens g, g + 8 for heads 2*q4, 2*q4 + 1
            const bool ok_lo = g < n_valid, ok_hi = g + 8 < n_valid;
            const float t0 = ok_lo ? sc[0] * p.scale_log2 : -INFINITY;
            const float t1 = ok_lo ? sc[1] * p.scale_log2 : -INFINITY;
            const float t2 = ok_hi ? sc[2] * p.scale_log2 : -INFINITY;
            const float t3 = ok_hi ? sc[3] * p.scale_log2 : -INFINITY;
            float mx0 = fmaxf(t0, t2), mx1 = fmaxf(t1, t3);
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
            }
            const float mn0 = fmaxf(m2[0], mx0), mn1 = fmaxf(m2[1], mx1);
            const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
            const float a0 = fast_exp2(m2[0] - ref0), a1 = fast_exp2(m2[1] - ref1);
            const float p0 = fast_exp2(t0 - ref0), p1 = fast_exp2(t1 - ref1);
            const float p2 = fast_exp2(t2 - ref0), p3 = fast_exp2(t3 - ref1);
            l[0] = l[0] * a0 + p0 + p2;
            l[1] = l[1] * a1 + p1 + p3;
            m2[0] = mn0;
            m2[1] = mn1;
            if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    o_acc[mt][0] *= a0;
                    o_acc[mt][1] *= a1;
                    o_acc[mt][2] *= a0;
                    o_acc[mt][3] *= a1;
                }
            }
            // P as the B operand [k = token][n = head]: transpose the C-fragment pairs across the warp
            const uint32_t b0 = movmatrix_trans(pack2<kBf16>(p0, p1));
            const uint32_t b1 = movmatrix_trans(pack2<kBf16>(p2, p3));
            // O^T += V^T . P
            const uint32_t v_row = tile + kTileBytes + v_tok * (kD * 2);
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, v_row + (((2 * mt + v_cc0) ^ lm_r) << 4));
                mma_16816<kBf16>(o_acc[mt], a, b0, b1);
            }
        }
        ++it;

        if (!st.seg_end) {
            continue;
        }

        // -- the pair ends inside this span: merge the warps, then publish ---------------------------------
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            l[0] += __shfl_xor_sync(0xffffffffu, l[0], o);
            l[1] += __shfl_xor_sync(0xffffffffu, l[1], o);
        }
        if (g == 0) {
            red_ml[(warp * kMaxGroup + 2 * q4) * 2 + 0] = m2[0];
            red_ml[(warp * kMaxGroup + 2 * q4) * 2 + 1] = l[0];
            red_ml[(warp * kMaxGroup + 2 * q4 + 1) * 2 + 0] = m2[1];
            red_ml[(warp * kMaxGroup + 2 * q4 + 1) * 2 + 1] = l[1];
        }
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int head = 2 * q4 + (e & 1);
                if (head < p.group) {
                    red_o[(warp * p.group + head) * kD + mt * 16 + g + 8 * (e >> 1)] = o_acc[mt][e];
                }
            }
        }
        __syncthreads();

        const int pair = st.s * p.nkvh + st.kvh;
        const long long pair_off = (long long)cum[st.s] * p.nkvh + (long long)st.kvh * (cum[st.s + 1] - cum[st.s]);
        const int pair_np = cum[st.s + 1] - cum[st.s];
        const int c_first = int(pair_off / span), c_last = int((pair_off + pair_np - 1) / span);
        const int expected = c_last - c_first + 1;
        float *slot = p.partials + (long long)(blockIdx.x + pair) * p.group * (kD + 2);

        // thread `tid` owns output dimension `tid` of every head of the group
        for (int h = 0; h < p.group; ++h) {
            float m_all = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                m_all = fmaxf(m_all, red_ml[(w * kMaxGroup + h) * 2]);
            }
            float l_all = 0.f, o = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float mw = red_ml[(w * kMaxGroup + h) * 2];
                const float wgt = mw == -INFINITY ? 0.f : fast_exp2(mw - m_all);
                l_all += red_ml[(w * kMaxGroup + h) * 2 + 1] * wgt;
                o += red_o[(w * p.group + h) * kD + tid] * wgt;
            }
            if (expected == 1) {
                const long long row = (long long)st.s * p.nh + st.kvh * p.group + h;
                const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
                if (p.part != nullptr) {
                    p.part[row * (kD + 2) + tid] = o * inv;
                    if (tid == 0) {
                        p.part[row * (kD + 2) + kD] = m_all * 0.6931471805599453f; // log2 units -> natural log
                        p.part[row * (kD + 2) + kD + 1] = l_all;
                    }
                } else {
                    store_out<kBf16>(p.out, row * kD + tid, o * inv);
                }
            } else {
                slot[h * (kD + 2) + tid] = o; // un-normalised, relative to m_all
                if (tid == 0) {
                    slot[h * (kD + 2) + kD] = m_all;
                    slot[h * (kD + 2) + kD + 1] = l_all;
                }
            }
        }

        if (expected > 1) {
            __syncthreads(); // every thread's partial is written
            if (tid == 0) {
                __threadfence(); // cumulative: publishes the CTA's partial device-wide before the arrival counts
                const int before = atomicAdd(&p.counters[pair], 1);
                s_last = (before == expected - 1) ? 1 : 0;
                __threadfence(); // the other CTAs' partials are visible to this CTA's reads below
            }
            __syncthreads();
            if (s_last) {
                const float *first = p.partials + (long long)(c_first + pair) * p.group * (kD + 2);
                combine_partials<kBf16>(first, expected, p.group, tid, red_o, [] { __syncthreads(); }, p.out, p.part,
                                        (long long)st.s * p.nh + st.kvh * p.group);
                if (tid == 0) {
                    p.counters[pair] = 0; // ready for the next launch
                }
            }
        }
        reset_state();
        new_pair = true;
        // red_o / red_ml are rewritten at the earliest after the next stage's __syncthreads
    }
    cp_async_wait<0>();
}

// ---- host side --------------------------------------------------------------------------------------

size_t smem_bytes(int group, int n_seqs) {
    return size_t(kRingBytes) + size_t(kWarps) * group * kD * sizeof(float) + size_t(kWarps) * kMaxGroup * 2 * sizeof(float) +
           size_t(n_seqs + 1) * sizeof(int);
}

template <bool kBf16>
void launch(cudaStream_t s, const DecodeParams &p, int grid, size_t smem) {
    static std::once_flag once[64];
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    std::call_once(once[dev & 63], [dev] {
        // opt in to the device's full per-block shared memory, less what the kernel holds statically
        int optin = 0;
        LLAISYS_CUDA_CHECK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        cudaFuncAttributes attr{};
        LLAISYS_CUDA_CHECK(cudaFuncGetAttributes(&attr, paged_decode_split_kernel<kBf16>));
        LLAISYS_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_split_kernel<kBf16>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                optin - int(attr.sharedSizeBytes)));
    });
    paged_decode_split_kernel<kBf16><<<grid, kThreads, smem, s>>>(p);
}

} // namespace

namespace {
int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        int n = 0;
        LLAISYS_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        return n;
    }
    if (cached[dev] == 0) {
        LLAISYS_CUDA_CHECK(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
    }
    return cached[dev];
}

} // namespace

int decode_grid_size(int32_t n_seqs, int32_t nkvh, int32_t max_kv_len) {
    const long long pages_bound = (long long)n_seqs * nkvh * ((max_kv_len + kPage - 1) / kPage);
    const long long by_work = (pages_bound + kPagesPerStage - 1) / kPagesPerStage; // at least one stage per CTA
    // Few (sequence, kv-head) pairs: every CTA that cuts a pair adds a partial result, and the pair's last CTA merges
    // them four per dependent round trip (about a microsecond each). With P pairs and H page-heads of 8 KiB, n CTAs
    // stream for about H * 8 KiB / (n * 22 GB/s) and merge for about n / (4 P) us: least near n = sqrt(1.5 P H); swept on
    // one to four sequences of 4096 to 131072 tokens, sqrt(P H) measured best (17 / 29 / 44 us for one sequence of 16384 /
    // 65536 / 131072 tokens).
    // Measured on one 16384-token sequence: 47.8 us with the full grid, 19.4 us with 64 CTAs. Batches with many pairs
    // reach the cap as before.
    const double balanced = std::sqrt(1.0 * double(n_seqs) * double(nkvh) * double(pages_bound));
    const long long by_merge = (long long)std::ceil(balanced);
    const long long cap = (long long)kCtasPerSm * sm_count();
    const long long want = by_work < by_merge ? by_work : by_merge;
    return int(want < 1 ? 1 : (want < cap ? want : cap));
}


void attention_decode_split_scratch(int32_t n_seqs, int32_t nh, int32_t nkvh, int32_t d, int32_t max_kv_len,
                                    size_t *partials_floats, size_t *counters_len) {
    *partials_floats = 0;
    *counters_len = 0;
    if (n_seqs <= 0 || nkvh <= 0 || nh <= 0 || d != kD || nh % nkvh != 0) {
        return;
    }
    const int grid = decode_grid_size(n_seqs, nkvh, max_kv_len);
    const size_t n_pairs = size_t(n_seqs) * nkvh;
    // the TMA kernel pads rows to 132 floats and keeps five more slots per CTA for merges that its warps share
    *partials_floats = (size_t(grid) * 6 + n_pairs) * size_t(nh / nkvh) * (kD + 4);
    *counters_len = n_pairs;
}

int attention_decode_split(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                           const void *q, float scale, const AttnOut &out, const AttnScratch &scratch) {
    const bool bf16 = dtype == LLAISYS_DTYPE_BF16;
    if (!(bf16 || dtype == LLAISYS_DTYPE_F16) || kv.d != kD || kv.page_size != kPage || kv.nkvh <= 0 ||
        batch.nh % kv.nkvh != 0 || batch.nh / kv.nkvh > kMaxGroup || batch.q_starts != nullptr ||
        batch.const_q_len != 1 || batch.n_seqs <= 0 || batch.n_seqs > kMaxSeqs) {
        return -1;
    }
    const int group = batch.nh / kv.nkvh;
    const int grid = decode_grid_size(batch.n_seqs, kv.nkvh, batch.max_kv_len);
    const size_t n_pairs = size_t(batch.n_seqs) * kv.nkvh;
    if (scratch.partials == nullptr || scratch.counters == nullptr || scratch.error_flag == nullptr ||
        scratch.partials_floats < (size_t(grid) + n_pairs) * group * (kD + 2) || scratch.counters_len < n_pairs) {
        return -1;
    }
    // 16-byte copies need 16-byte aligned rows on the K/V side
    if ((kv.page_stride * 2) % 16 || (kv.head_stride * 2) % 16 || (kv.token_stride * 2) % 16 ||
        reinterpret_cast<uintptr_t>(kv.k_base) % 16 || reinterpret_cast<uintptr_t>(kv.v_base) % 16 ||
        reinterpret_cast<uintptr_t>(q) % 4) {
        return -1;
    }
    DecodeParams p;
    p.k_base = static_cast<const char *>(kv.k_base);
    p.v_base = static_cast<const char *>(kv.v_base);
    p.page_stride_b = kv.page_stride * 2;
    p.head_stride_b = kv.head_stride * 2;
    p.token_stride_b = kv.token_stride * 2;
    p.block_table = kv.block_table;
    p.table_stride = kv.table_stride;
    p.num_pages = kv.num_pages;
    // a sequence can never be longer than its block table (paged) or the tensor (contiguous)
    p.max_tokens = kv.block_table ? kv.table_stride * kPage : batch.max_kv_len;
    p.seq_ids = batch.seq_ids;
    p.kv_lens = batch.kv_lens;
    p.const_kv_len = batch.const_kv_len;
    p.n_seqs = batch.n_seqs;
    p.nkvh = kv.nkvh;
    p.group = group;
    p.nh = batch.nh;
    p.q = q;
    p.out = out.out;
    p.part = out.part;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.partials = scratch.partials;
    p.counters = scratch.counters;
    p.error_flag = scratch.error_flag;
    const size_t smem = smem_bytes(group, batch.n_seqs);
    auto s = static_cast<cudaStream_t>(stream);
    if (bf16) {
        launch<true>(s, p, grid, smem);
    } else {
        launch<false>(s, p, grid, smem);
    }
    check_launch("paged_decode_split");
    return 0;
}

} // namespace llaisys::kernels
