// K4: chunked-prefill attention over the page pool on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Roofline: tensor. Algorithmic flops per sequence = 4 * nh * d * sum over chunk rows of visible keys
//                                                  = 4 * nh * 128 * (L * C + L * (L + 1) / 2)
// for a chunk of L queries after C cached tokens (QK^T and PV, 2 flops per multiply-add; masked work not counted).
//
// One CTA per (sequence, query head, block of 128 chunk rows). Its 128 query rows stay in shared memory for the
// whole tile; K/V arrive 64 tokens (4 pages) at a time:
//   warp 4 (producer)  reads the block table and issues TMA tiles (16 tokens x 64 dims, 128-byte swizzle) into a
//                      two-stage K/V ring -- K as [2 dim-halves][64 tokens][128 B], V the same;
//   warp 5 (MMA)       one thread issues tcgen05.mma (M 128, K 16, bf16/f16 -> f32):
//                        S = Q . K^T      N 64, 8 instructions, both operands K-major, accumulator S[buf] in TMEM
//                        O += P . V       N 128, 4 instructions, P K-major from shared memory, V MN-major (the page layout
//                                         keeps head_dim contiguous), accumulator O in TMEM
//                      QK^T of block i+1 is issued before PV of block i, so the tensor pipe works under the softmax;
//   warps 0-3          the 128 softmax threads, one query row each (TMEM lane = row): tcgen05.ld S in 32-column
//                      pieces, causal mask, running max / sum in the log2 domain, P = 2^(s - m) written to shared
//                      memory as bf16 in the swizzled K-major layout, O rescaled in TMEM only when a row's max grew by
//                      more than 2^8 since the last rescale (the stale max is used consistently for P and the sum).
// TMEM: 256 columns per CTA: S double-buffered (2 x 64) + O (128). Shared memory: Q 32 KiB + P 16 KiB + K/V
// 2 x 32 KiB = 112 KiB, so TWO CTAs share an SM (and its 512 TMEM columns): while one CTA's 128 softmax threads work
// on a block, the other CTA's MMAs keep the tensor pipe busy. Tiles are handed out longest sequence first.
//
// Synchronisation is mbarriers only; tcgen05.commit arrives on them when the tensor pipe has finished. Every wait is
// bounded: a wait that runs out sets bit 8 of the error word and the CTA winds down (TMEM is freed) instead of hanging.
// No cluster launch, no multicast.
#include "kernels.hpp"
#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"

#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace llaisys::kernels {

namespace {

constexpr int kD = 128;
constexpr int kPage = 16;
constexpr int kBlockM = 128;                 // query rows per CTA
constexpr int kBlockN = 64;                  // keys per K/V block (4 pages)
constexpr int kPagesPerBlock = kBlockN / kPage;
constexpr int kStages = 2;
constexpr int kSoftmaxThreads = 128;
constexpr int kProducerWarp = 4, kMmaWarp = 5;
constexpr int kThreads = 192;
// Every operand is stored as 64-element (128-byte) column halves of [rows][128 B], 128-byte swizzled.
constexpr int kQHalfBytes = kBlockM * 128;       // Q: 128 rows x 64 dims, 16 KiB; two of them
constexpr int kQBytes = 2 * kQHalfBytes;
constexpr int kPHalfBytes = kBlockM * 128;       // P: 128 rows x 64 keys
constexpr int kPBytes = (kBlockN / 64) * kPHalfBytes;
constexpr int kKvHalfBytes = kBlockN * 128;      // K (or V): kBlockN keys x 64 dims; two of them per operand
constexpr int kKvOperandBytes = 2 * kKvHalfBytes;
constexpr int kStageBytes = 2 * kKvOperandBytes; // K block + V block
constexpr int kTmemCols = 256;                   // per CTA; two CTAs share the SM's 512 columns
constexpr int kColS = 0, kColO = 2 * kBlockN;    // S buffers at columns 0 and kBlockN, O (128 columns) after them
constexpr int kAlignSlack = 256;                 // spare bytes in front of the operands (two CTAs must fit one SM)
constexpr int kMaxSortedSeqs = 256;              // batches up to this size are scheduled longest sequence first
static_assert(kBlockN % 64 == 0 && kColO + kD <= kTmemCols, "TMEM budget");
constexpr int kErrTimeout = 8;
constexpr float kRescaleThreshold = 8.f;     // log2 units

// barrier indices
enum : int {
    kBarKFull = 0,                    // [kStages] producer -> MMA: K block landed (transaction bytes)
    kBarKEmpty = kBarKFull + kStages, // [kStages] MMA (commit) -> producer: QK^T of the block finished
    kBarVFull = kBarKEmpty + kStages, // [kStages] producer -> MMA: V block landed
    kBarVEmpty = kBarVFull + kStages, // [kStages] MMA (commit) -> producer: PV of the block finished
    kBarSFull = kBarVEmpty + kStages, // [2] MMA (commit) -> softmax: S[buf] written
    kBarSFree = kBarSFull + 2,          // [2] softmax (128) -> MMA: S[buf] read
    kBarPFull = kBarSFree + 2,          // softmax (128) -> MMA: P in shared memory, O rescaled
    kBarPFree = kBarPFull + 1,          // MMA (commit) -> softmax: PV finished: P reusable, O stable
    kNumBars = kBarPFree + 1
};

struct PrefillParams {
    long long page0;
    const int32_t *block_table;
    int32_t table_stride, num_pages;
    const int32_t *seq_ids;
    const int32_t *kv_lens;
    const int32_t *q_starts; // [n_seqs + 1]; null in contiguous mode
    int32_t contiguous;      // 1: K and V are plain [tokens, nkvh, 128] tensors of ONE sequence (no block table, two
                             // 3-D tensor maps); q rows [0, const_q_len), const_kv_len keys
    int32_t const_q_len, const_kv_len;
    int32_t n_seqs, nkvh, group, nh, q_blocks; // q_blocks = ceil(max_q_len / 128)
    const void *q;
    void *out;
    float scale_log2;
    int32_t *error_flag;
};

// kPTmem: P goes from the softmax threads to the PV product through tensor memory (packed 16-bit pairs written over
// the first 32 columns of the S buffer they were computed from, read back as the A operand) instead of through shared
// memory: per 64-key block this takes a 16 KiB store and a 16 KiB operand read off the shared-memory port (which also
// carries 32 KiB of TMA writes, 48 KiB of QK^T operand reads and 16 KiB of V reads) and the proxy fence out of the
// softmax-to-tensor-pipe chain. Consecutive P tiles sit in alternate S buffers; QK^T of block i + 2, which overwrites
// the buffer of P(i), is issued after PV of block i.
template <bool kBf16, bool kPTmem>
__global__ void __launch_bounds__(kThreads, 2)
    paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_v,
                            PrefillParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t base_u32 = (raw_u32 + 1023u) & ~1023u; // swizzled operands need 1 KiB alignment
    unsigned char *base = smem_raw + (base_u32 - raw_u32);
    const uint32_t q_u32 = base_u32, p_u32 = base_u32 + kQBytes, kv_u32 = base_u32 + kQBytes + kPBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + kQBytes + kPBytes + kStages * kStageBytes);
    const uint32_t bars_u32 = smem_u32(bars);
    uint32_t *s_tmem_base = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem_base + 1);
    int16_t *s_order = reinterpret_cast<int16_t *>(s_tmem_base + 2); // [min(n_seqs, kMaxSortedSeqs)]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (base_u32 - raw_u32 > uint32_t(kAlignSlack)) { // cannot place the swizzled operands: report, do not run
        if (tid == 0) {
            atomicOr(p.error_flag, kErrTimeout);
        }
        return;
    }

    // ---- which tile: sequences by decreasing length (the order CTAs are handed out is the order they start) ------
    const bool sorted = p.n_seqs <= kMaxSortedSeqs && !p.contiguous;
    if (sorted) {
        for (int a = tid; a < p.n_seqs; a += kThreads) {
            const int len_a = p.kv_lens[a];
            int rank = 0;
            for (int b = 0; b < p.n_seqs; ++b) {
                const int len_b = p.kv_lens[b];
                rank += (len_b > len_a || (len_b == len_a && b < a)) ? 1 : 0;
            }
            s_order[rank] = int16_t(a);
        }
    }
    __syncthreads();
    const int linear = blockIdx.x;
    const int per_seq = p.q_blocks * p.nh;
    const int s = sorted ? int(s_order[linear / per_seq]) : linear / per_seq;
    const int within = linear % per_seq;
    const int qb = p.q_blocks - 1 - within / p.nh; // late query blocks see the most keys: first
    const int h = within % p.nh;
    const int q_start = p.contiguous ? 0 : p.q_starts[s];
    const int q_len = p.contiguous ? p.const_q_len : p.q_starts[s + 1] - q_start;
    if (qb * kBlockM >= q_len) {
        return; // uniform over the CTA, before any mbarrier or TMEM allocation
    }
    const int kv_len = p.contiguous ? max(p.const_kv_len, q_len) : min(max(p.kv_lens[s], q_len), p.table_stride * kPage);
    const int off = kv_len - q_len;                                   // query t sees keys j <= t + off
    const int kv_hi = min(kv_len, qb * kBlockM + kBlockM + off);      // keys any row of this tile can see
    const int nblk = (kv_hi + kBlockN - 1) / kBlockN;
    const int n_pages = (kv_hi + kPage - 1) / kPage;
    const int kvh = h / p.group;
    const int seq_row = (!p.contiguous && p.seq_ids) ? p.seq_ids[s] : s;

    // ---- set-up: barriers, TMEM, Q tile, cleared K/V ring ---------------------------------------------------
    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            const bool many = (i >= kBarSFree && i < kBarSFree + 2) || i == kBarPFull;
            mbar_init(bars_u32 + i * 8, many ? kSoftmaxThreads : 1);
        }
        *s_abort = 0;
        mbar_init_fence();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(s_tmem_base), kTmemCols);
        tmem_relinquish();
    }
    {
        // Q rows of this tile, 16 bytes per store, into the K-major 128-byte-swizzled layout
        // [dims 0-63 | dims 64-127][128 rows][128 B]; rows past the chunk are zero.
        const char *q_base = static_cast<const char *>(p.q);
        for (int idx = tid; idx < kBlockM * 16; idx += kThreads) {
            const int r = idx >> 4, cc = idx & 15;
            const int t = qb * kBlockM + r;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (t < q_len) {
                val = *reinterpret_cast<const uint4 *>(q_base + ((long long)(q_start + t) * p.nh + h) * (kD * 2) + cc * 16);
            }
            const uint32_t dst = q_u32 + (cc >> 3) * kQHalfBytes + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w) : "memory");
        }
        // A block shorter than kBlockN keys leaves ring rows unwritten; they are masked out of S, but V rows enter
        // the PV product with weight 0, so they must at least be finite: start from zeros.
        for (int idx = tid; idx < kStages * kStageBytes / 16; idx += kThreads) {
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(kv_u32 + idx * 16), "r"(0u) : "memory");
        }
        fence_proxy_async_smem(); // generic-proxy stores above are read (Q) or overwritten (ring) by the async proxy
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;

    auto bar = [&](int which) { return bars_u32 + uint32_t(which) * 8; };
    auto give_up = [&]() {
        *s_abort = 1;
        atomicOr(p.error_flag, kErrTimeout);
    };

    if (warp == kProducerWarp) {
        // ================================ producer: TMA tiles of K and V =====================================
        const long long tbase = (long long)seq_row * p.table_stride;
        // K and V of a block have separate barriers: the K slot is free again as soon as QK^T of its block is done,
        // one whole block earlier than the V slot (PV runs after the softmax), so K of block i + 2 is in flight early
        // enough to hide the copy latency with only two stages.
        bool alive = true;
        for (int i = 0; i < nblk && alive; ++i) {
            const int st = i & 1;
            const int first = i * kPagesPerBlock;
            const int n_pg = min(kPagesPerBlock, n_pages - first);
            int page = 0;
            if (lane < n_pg) {
                if (p.contiguous) {
                    page = first + lane; // block b of the tensor is its tokens [16 b, 16 b + 16)
                } else {
                    page = p.block_table[tbase + first + lane];
                    if (page < 0 || page >= p.num_pages) {
                        atomicOr(p.error_flag, kErrBadPage);
                        page = 0;
                    }
                }
            }
            const int c3 = int((p.page0 + page) * 2);
            const uint32_t dst = kv_u32 + st * kStageBytes + lane * 2048;
#pragma unroll
            for (int is_v = 0; is_v < 2; ++is_v) {
                const int full = (is_v ? kBarVFull : kBarKFull) + st, empty = (is_v ? kBarVEmpty : kBarKEmpty) + st;
                if (i >= kStages && !wait_or_abort(bar(empty), uint32_t((i >> 1) - 1) & 1u, s_abort)) {
                    if (lane == 0) {
                        give_up();
                    }
                    alive = false;
                    break;
                }
                if (lane == 0) {
                    mbar_arrive_expect_tx(bar(full), uint32_t(n_pg) * 2 * 2048);
                }
                __syncwarp();
                if (lane < n_pg) {
                    const uint32_t lo = dst + is_v * kKvOperandBytes, hi = lo + kKvHalfBytes; // dims 0-63, dims 64-127
                    if (p.contiguous) {
                        // [tokens][kv-heads][128] tensors: box = 64 dims x 1 head x 16 tokens; tokens past the end read as 0
                        const CUtensorMap *m = is_v ? &tmap_v : &tmap;
                        tma_load_3d(lo, m, 0, kvh, page * kPage, bar(full));
                        tma_load_3d(hi, m, 64, kvh, page * kPage, bar(full));
                    } else {
                        tma_load_4d(lo, &tmap, 0, 0, kvh, c3 + is_v, bar(full));
                        tma_load_4d(hi, &tmap, 64, 0, kvh, c3 + is_v, bar(full));
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ================================ MMA issuer (one thread) =============================================
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(kBf16, false, kBlockM, kBlockN);
            constexpr uint32_t idesc_pv = make_idesc(kBf16, true, kBlockM, kD);
            const uint32_t tmem_o = tmem_base + kColO;
            bool ok = true;
            auto issue_pv = [&](int j) { // O (+)= P . V of block j
                if (!wait_or_abort(bar(kBarPFull), uint32_t(j) & 1u, s_abort) ||
                    !wait_or_abort(bar(kBarVFull + (j & 1)), uint32_t(j >> 1) & 1u, s_abort)) {
                    return false;
                }
                tc_fence_after();
                const uint32_t v_u32 = kv_u32 + (j & 1) * kStageBytes + kKvOperandBytes;
#pragma unroll
                for (int kk = 0; kk < kBlockN / 16; ++kk) {
                    // B = 16 keys x 128 dims of V, MN-major: 8-key groups 1 KiB apart, the two 64-dim halves one
                    // half-operand apart
                    const uint64_t b = smem_desc_sw128(v_u32 + kk * 2048, kKvHalfBytes, 1024);
                    if constexpr (kPTmem) {
                        // A = P rows x 16 keys from tensor memory: 8 columns of packed pairs per step, in S buffer j & 1
                        umma_f16_ts(tmem_o, tmem_base + kColS + (j & 1) * kBlockN + kk * 8, b, idesc_pv,
                                    (j > 0 || kk > 0) ? 1u : 0u);
                        continue;
                    }
                    // A = P rows x 16 keys (K-major: 32 bytes into the 128-byte row per step, next half after 4 steps)
                    const uint64_t a = smem_desc_sw128(p_u32 + (kk >> 2) * kPHalfBytes + (kk & 3) * 32, 0, 1024);
                    umma_f16(tmem_o, a, b, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(bar(kBarPFree));
                umma_commit(bar(kBarVEmpty + (j & 1)));
                return true;
            };
            for (int i = 0; i < nblk && ok; ++i) {
                const int st = i & 1, buf = i & 1;
                ok = wait_or_abort(bar(kBarKFull + st), uint32_t(i >> 1) & 1u, s_abort);
                if (ok && i >= 2) {
                    ok = wait_or_abort(bar(kBarSFree + buf), uint32_t((i >> 1) - 1) & 1u, s_abort);
                }

                if (!ok) {
                    break;
                }
                tc_fence_after();
                const uint32_t k_u32 = kv_u32 + st * kStageBytes;
#pragma unroll
                for (int ks = 0; ks < kD / 16; ++ks) {
                    const uint64_t a = smem_desc_sw128(q_u32 + (ks >> 2) * kQHalfBytes + (ks & 3) * 32, 0, 1024);
                    const uint64_t b = smem_desc_sw128(k_u32 + (ks >> 2) * kKvHalfBytes + (ks & 3) * 32, 0, 1024);
                    umma_f16(tmem_base + kColS + buf * kBlockN, a, b, idesc_qk, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(kBarSFull + buf));
                umma_commit(bar(kBarKEmpty + st));
                if (i >= 1) {
                    ok = issue_pv(i - 1);
                }
            }
            if (ok) {
                ok = issue_pv(nblk - 1);
            }
            if (!ok) {
                give_up();
            }
        }
    } else {
        // ================================ softmax: one query row per thread =====================================
        const int row = tid;                       // TMEM lane
        const int t = qb * kBlockM + row;          // query index inside the chunk
        const int last_visible = t + off;          // keys j <= last_visible (and < kv_len) take part
        const uint32_t lane_base = uint32_t(warp * 32) << 16;
        const uint32_t tmem_o = tmem_base + lane_base + kColO;
        float m_used = -INFINITY, l = 0.f;
        bool dead = false;
        for (int i = 0; i < nblk && !dead; ++i) {
            const int buf = i & 1;
            if (!wait_or_abort(bar(kBarSFull + buf), uint32_t(i >> 1) & 1u, s_abort)) {
                dead = true;
                break;
            }
            tc_fence_after();
            const uint32_t tmem_s = tmem_base + lane_base + kColS + buf * kBlockN;
            const int j0 = i * kBlockN;
            const int n_ok = min(min(last_visible, kv_len - 1) - j0 + 1, kBlockN); // visible columns are [0, n_ok)
            // One TMEM read of the row's kBlockN scores; S[buf] is handed back to the tensor pipe straight away.
            uint32_t sr[kBlockN / 32][32];
#pragma unroll
            for (int c = 0; c < kBlockN / 32; ++c) {
                tmem_ld32_nowait(tmem_s + c * 32, sr[c]);
            }
            tmem_wait_ld();
            if constexpr (!kPTmem) {
                tc_fence_before();
                mbar_arrive(bar(kBarSFree + buf)); // S[buf] may be overwritten by QK^T of block i + 2
            }
            // Most blocks lie wholly below the diagonal: the whole warp then skips the mask (warp-uniform choice).
            const bool plain = __all_sync(0xffffffffu, n_ok >= kBlockN) && p.scale_log2 > 0.f;
            // Row maximum as eight independent chains (a single chain of 64 dependent max operations would cost more than
            // the exponentials that follow).
            float mx8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                mx8[u] = -INFINITY;
            }
            if (plain) {
#pragma unroll
                for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                        mx8[k & 7] = fmaxf(mx8[k & 7], __uint_as_float(sr[c][k]));
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                        if (c * 32 + k < n_ok) {
                            mx8[k & 7] = fmaxf(mx8[k & 7], __uint_as_float(sr[c][k]) * p.scale_log2);
                        }
                    }
                }
            }
            float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                             fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            if (plain) {
                mx *= p.scale_log2;
            }
            // The running max only moves when it grew by more than 2^8: P and the row sum both use m_used, so the
            // result is exact either way, and O is rescaled rarely.
            float alpha = 1.f;
            const bool grow = mx > m_used + kRescaleThreshold;
            if (grow) {
                alpha = fast_exp2(m_used - mx); // 0 on the first block
                m_used = mx;
            }
            l *= alpha;
            // P = 2^(s - m) as 16-bit, computed into registers BEFORE waiting for the previous PV: only the stores of
            // P sit on the block-to-block dependency chain.
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            uint32_t packed[kBlockN / 2];
            float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f; // independent sums: short dependency chains
            if (plain) {
#pragma unroll
                for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                    for (int k = 0; k < 32; k += 2) {
                        const float x0 = fmaf(__uint_as_float(sr[c][k]), p.scale_log2, neg_m);
                        const float x1 = fmaf(__uint_as_float(sr[c][k + 1]), p.scale_log2, neg_m);
                        // (computing a share of these on the FMA pipe with a polynomial was measured: 1 to 3 pairs of every
                        // 8 made the kernel 2 to 8 % slower -- the softmax warps are short of issue slots, not of MUFU rate)
                        const float p0 = fast_exp2(x0);
                        const float p1 = fast_exp2(x1);
                        if (k & 2) {
                            l2 += p0;
                            l3 += p1;
                        } else {
                            l0 += p0;
                            l1 += p1;
                        }
                        packed[c * 16 + (k >> 1)] = pack2<kBf16>(p0, p1);
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                    for (int k = 0; k < 32; k += 2) {
                        const float p0 = (c * 32 + k < n_ok) ? fast_exp2(fmaf(__uint_as_float(sr[c][k]), p.scale_log2, neg_m)) : 0.f;
                        const float p1 =
                            (c * 32 + k + 1 < n_ok) ? fast_exp2(fmaf(__uint_as_float(sr[c][k + 1]), p.scale_log2, neg_m)) : 0.f;
                        l0 += p0;
                        l1 += p1;
                        packed[c * 16 + (k >> 1)] = pack2<kBf16>(p0, p1);
                    }
                }
            }
            l += (l0 + l1) + (l2 + l3);
            // PV of the previous block must be finished before O is rescaled and, on the shared-memory path, before P is
            // overwritten. With P in tensor memory the hand-over itself would not need this wait, but every phase of the
            // barrier has to be observed in order: a parity wait cannot tell "two phases behind" from "done", and a
            // thread that skipped phases passed the final wait before the last two products had finished (rare wrong
            // rows in tiles that ran alone on their SM).
            const bool any_grow = __any_sync(0xffffffffu, grow);
            if (i >= 1) {
                if (!wait_or_abort(bar(kBarPFree), uint32_t(i - 1) & 1u, s_abort)) {
                    dead = true;
                    break;
                }
                tc_fence_after();
                if (any_grow) {
#pragma unroll
                    for (int c = 0; c < kD / 32; ++c) {
                        float v[32];
                        tmem_ld32(tmem_o + c * 32, v);
#pragma unroll
                        for (int k = 0; k < 32; ++k) {
                            v[k] *= alpha;
                        }
                        tmem_st32(tmem_o + c * 32, v);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                }
            }
            if constexpr (kPTmem) {
                // 64 keys = 32 columns of packed pairs over the first half of S[buf]; the same arrival tells the tensor
                // pipe that P is there and (S having been read above) that the buffer may be rewritten after this PV
                tmem_st32_words(tmem_s, packed);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar(kBarSFree + buf));
                mbar_arrive(bar(kBarPFull));
                continue;
            }
#pragma unroll
            for (int cc = 0; cc < kBlockN / 8; ++cc) { // 16-byte chunk (8 keys) of this row, swizzled K-major layout
                const uint32_t dst = p_u32 + (cc >> 3) * kPHalfBytes + row * 128 + (((cc & 7) ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "r"(packed[cc * 4]),
                             "r"(packed[cc * 4 + 1]), "r"(packed[cc * 4 + 2]), "r"(packed[cc * 4 + 3])
                             : "memory");
            }
            fence_proxy_async_smem(); // P stores -> visible to the tensor pipe's reads
            mbar_arrive(bar(kBarPFull));
        }
        // ---- epilogue: O / l -> out ------------------------------------------------------------------------------
        if (!dead && !wait_or_abort(bar(kBarPFree), uint32_t(nblk - 1) & 1u, s_abort)) {
            dead = true;
        }
        if (dead) {
            if (lane == 0) {
                give_up();
            }
        } else {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            char *out_row = static_cast<char *>(p.out) + ((long long)(q_start + t) * p.nh + h) * (kD * 2);
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                float v[32];
                tmem_ld32(tmem_o + c4 * 32, v);
                if (t < q_len) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 w;
                        w.x = pack2<kBf16>(v[q4 * 8 + 0] * inv, v[q4 * 8 + 1] * inv);
                        w.y = pack2<kBf16>(v[q4 * 8 + 2] * inv, v[q4 * 8 + 3] * inv);
                        w.z = pack2<kBf16>(v[q4 * 8 + 4] * inv, v[q4 * 8 + 5] * inv);
                        w.w = pack2<kBf16>(v[q4 * 8 + 6] * inv, v[q4 * 8 + 7] * inv);
                        *reinterpret_cast<uint4 *>(out_row + c4 * 64 + q4 * 16) = w;
                    }
                }
            }
        }
    }

    // ---- teardown: everyone is done with TMEM before the allocating warp frees it ----------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

} // namespace

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn prefill_encode_fn() {
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

// operands + barriers + TMEM-address / abort words + sequence order; kAlignSlack bytes for the 1 KiB alignment of the
// operand area (the dynamic window itself starts aligned when the kernel has no static shared memory)
constexpr size_t kSmemBytes = kAlignSlack + kQBytes + kPBytes + kStages * kStageBytes + kNumBars * sizeof(uint64_t) + 8 +
                              kMaxSortedSeqs * sizeof(int16_t);

template <bool kBf16, bool kPTmem>
void launch_variant(cudaStream_t s, const CUtensorMap &tmap, const CUtensorMap &tmap_v, const PrefillParams &p, int grid) {
    static std::once_flag once[64];
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    std::call_once(once[dev & 63], [] {
        LLAISYS_CUDA_CHECK(cudaFuncSetAttribute(paged_prefill_tc_kernel<kBf16, kPTmem>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)));
    });
    paged_prefill_tc_kernel<kBf16, kPTmem><<<grid, kThreads, kSmemBytes, s>>>(tmap, tmap_v, p);
}

template <bool kBf16>
void launch(cudaStream_t s, const CUtensorMap &tmap, const CUtensorMap &tmap_v, const PrefillParams &p, int grid) {
    // LLAISYS_PREFILL_P=smem keeps P on the shared-memory path (the earlier design), for comparison
    static const bool p_tmem = [] {
        const char *e = std::getenv("LLAISYS_PREFILL_P");
        return e == nullptr || std::string(e) != "smem";
    }();
    if (p_tmem) {
        launch_variant<kBf16, true>(s, tmap, tmap_v, p, grid);
    } else {
        launch_variant<kBf16, false>(s, tmap, tmap_v, p, grid);
    }
}

} // namespace

int make_kv_tile_tensor_map(void *out_128_bytes, void *pool_base, uint64_t total_rows, uint32_t nkvh,
                            llaisysDataType_t dtype) {
    if (dtype != LLAISYS_DTYPE_BF16 && dtype != LLAISYS_DTYPE_F16) {
        return -1;
    }
    if (total_rows == 0 || nkvh == 0 || total_rows % (uint64_t(kPage) * nkvh) != 0 || total_rows >= (uint64_t(1) << 31) ||
        reinterpret_cast<uintptr_t>(pool_base) % 16 != 0) {
        return -1;
    }
    EncodeTiledFn encode = prefill_encode_fn();
    if (encode == nullptr) {
        return -1;
    }
    // Same 4-D view of the pool as the decode kernel's map -- [page-and-K|V][kv-head][slot][128 elements] -- with a
    // box of one half-tile: 64 elements x 16 slots (2 KiB, 128-byte swizzle).
    const cuuint64_t dims[4] = {cuuint64_t(kD), cuuint64_t(kPage), cuuint64_t(nkvh), cuuint64_t(total_rows / (kPage * nkvh))};
    const cuuint64_t strides[3] = {cuuint64_t(kD * 2), cuuint64_t(kPage * kD * 2), cuuint64_t(kPage * kD * 2) * nkvh};
    const cuuint32_t box[4] = {64, cuuint32_t(kPage), 1, 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    CUtensorMap map;
    const CUresult rc =
        encode(&map, dtype == LLAISYS_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
               pool_base, dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        return -1;
    }
    memcpy(out_128_bytes, &map, sizeof(map));
    return 0;
}

namespace {

// [tokens][nkvh][128] 16-bit tensor -> 3-D map (dims 128, nkvh, tokens) with a box of 64 dims x 1 head x 16 tokens: the
// tile lands in shared memory exactly like a page-pool tile; rows past the last token are out of bounds and read as 0.
bool contiguous_kv_map(CUtensorMap *out, const void *base, const KVView &kv, uint64_t tokens, bool bf16) {
    EncodeTiledFn encode = prefill_encode_fn();
    if (encode == nullptr || tokens == 0 || tokens >= (uint64_t(1) << 31)) {
        return false;
    }
    const cuuint64_t dims[3] = {cuuint64_t(kD), cuuint64_t(kv.nkvh), cuuint64_t(tokens)};
    const cuuint64_t strides[2] = {cuuint64_t(kv.head_stride) * 2, cuuint64_t(kv.token_stride) * 2};
    const cuuint32_t box[3] = {64, 1, cuuint32_t(kPage)};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    return encode(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base),
                  dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace

int attention_prefill_tc(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                         const void *q, float scale, const AttnOut &out, int32_t *error_flag) {
    const bool bf16 = dtype == LLAISYS_DTYPE_BF16;
    if (!(bf16 || dtype == LLAISYS_DTYPE_F16) || kv.d != kD || kv.page_size != kPage || kv.nkvh <= 0 || out.out == nullptr ||
        out.part != nullptr || batch.nh % kv.nkvh != 0 || batch.n_seqs <= 0 || batch.max_q_len <= 0 || error_flag == nullptr ||
        reinterpret_cast<uintptr_t>(q) % 16 != 0 || reinterpret_cast<uintptr_t>(out.out) % 16 != 0) {
        return -1;
    }
    // Two kinds of K/V: a page pool with a block table (one tensor map over the pool, made with the cache), or the
    // legacy operator's plain [tokens, nkvh, 128] tensors of one sequence (two maps made here).
    const bool paged = kv.block_table != nullptr;
    if (paged && (kv.tma_tile_desc == nullptr || batch.kv_lens == nullptr || batch.q_starts == nullptr)) {
        return -1;
    }
    const bool contiguous = !paged && batch.n_seqs == 1 && batch.q_starts == nullptr && batch.kv_lens == nullptr &&
                            batch.seq_ids == nullptr && batch.const_q_len > 1 && batch.const_kv_len >= batch.const_q_len &&
                            kv.head_stride == kD && kv.token_stride == int64_t(kv.nkvh) * kD &&
                            reinterpret_cast<uintptr_t>(kv.k_base) % 16 == 0 && reinterpret_cast<uintptr_t>(kv.v_base) % 16 == 0;
    if (!paged && !contiguous) {
        return -1;
    }
    PrefillParams p;
    p.page0 = paged ? kv.tma_page0 : 0;
    p.block_table = kv.block_table;
    p.table_stride = kv.table_stride;
    p.num_pages = kv.num_pages;
    p.seq_ids = batch.seq_ids;
    p.kv_lens = batch.kv_lens;
    p.q_starts = batch.q_starts;
    p.contiguous = contiguous ? 1 : 0;
    p.const_q_len = batch.const_q_len;
    p.const_kv_len = batch.const_kv_len;
    p.n_seqs = batch.n_seqs;
    p.nkvh = kv.nkvh;
    p.group = batch.nh / kv.nkvh;
    p.nh = batch.nh;
    p.q_blocks = (batch.max_q_len + kBlockM - 1) / kBlockM;
    p.q = q;
    p.out = out.out;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_flag = error_flag;
    const long long grid = (long long)batch.n_seqs * batch.nh * p.q_blocks;
    if (grid > 0x7fffffffLL) {
        return -1;
    }
    CUtensorMap tmap, tmap_v;
    if (paged) {
        memcpy(&tmap, kv.tma_tile_desc, sizeof(tmap));
        tmap_v = tmap;
    } else if (!contiguous_kv_map(&tmap, kv.k_base, kv, uint64_t(batch.const_kv_len), bf16) ||
               !contiguous_kv_map(&tmap_v, kv.v_base, kv, uint64_t(batch.const_kv_len), bf16)) {
        return -1;
    }
    auto s = static_cast<cudaStream_t>(stream);
    if (bf16) {
        launch<true>(s, tmap, tmap_v, p, int(grid));
    } else {
        launch<false>(s, tmap, tmap_v, p, int(grid));
    }
    check_launch("paged_prefill_tc");
    return 0;
}

} // namespace llaisys::kernels
