// K2 + K3 for the page pool, TMA edition: split-KV flash decoding with a warp-specialised copy pipeline.
//
// Same mathematics, work decomposition ("even page split" over persistent CTAs, two per SM) and fused
// log-sum-exp combine as attention_decode.cu; what changes is how K/V reach shared memory and who moves them:
//   * one PRODUCER warp per CTA walks the CTA's span of pages, reads the block table 32 entries at a time, and up
//     to 12 of its lanes issue the copies of a round in parallel: each (page, kv-head) is two 4 KiB boxes of one 4-D
//     tensor map over the pool, [page and K|V][kv-head][slot][128 elements] with box {64 dims, 16 slots, 1 head, K and
//     V} (cp.async.bulk.tensor.4d; low 64 dims, then high 64 dims), landing in one 8 KiB slot of a 12-slot ring with the
//     hardware 128-byte swizzle, completion counted on the slot's "full" mbarrier;
//   * a sixth EPILOGUE warp counts the CTAs that have finished a (sequence, kv-head) pair and, for the last one to
//     arrive, merges the pair's partial results (log-sum-exp combine) while the consumers go on;
//   * four CONSUMER warps take pages round-robin: wait on "full", 8 + 8 mma.sync m16n8k16 with conflict-free
//     ldmatrix reads (the swizzle XORs the 16-byte chunk index with token % 8), then hand the slot back through
//     its "empty" mbarrier. They execute ~100 instructions per page and never compute an address in global
//     memory, so the copy engine runs up to 96 KiB ahead of them per CTA (192 KiB per SM in flight).
// Measured motivation: the cp.async version spent its issue slots on address arithmetic and its time in
// long-scoreboard stalls behind block-table loads, reaching 45 % of DRAM throughput with 8 warps per SM.
//
// Fused step (k_new / v_new given): the call also appends one new K/V row per sequence, at position kv_len - 1, so a
// decode step is ONE launch. The consumer warp that takes a pair's last page fetches the pair's new row with cp.async
// while it loads q, writes it over its slot of the tile in shared memory once the page has landed (whatever the TMA copy
// read of that slot, old bytes or a torn new row, is replaced) and stores it into the page in global memory for later
// calls. Nobody else reads that row in this launch: a (page, kv-head) tile is copied by exactly one CTA.
//
// Every mbarrier wait is bounded; a wait that runs out sets bit 8 of the error word, the CTA stops touching the
// ring (its warps still meet at their named barriers) and the launch ends with wrong output and a flagged error
// instead of a hang. No cluster multicast is used anywhere.
#include "kernels.hpp"
#include "decode_epilogue.cuh"
#include "mma_utils.cuh"

#include <cuda.h>

#include <cstring>
#include <mutex>
#include <type_traits>

namespace llaisys::kernels {

namespace {

constexpr int kConsumerWarps = 4; // two CTAs per SM
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerWarp = kConsumerWarps;      // warp 4 issues the copies
constexpr int kEpilogueWarp = kConsumerWarps + 1;  // warp 5 counts arrivals and merges cut pairs
constexpr int kThreads = kConsumerThreads + 64;
constexpr int kSlots = 3 * kConsumerWarps;
constexpr int kIssueLanes = kSlots < 32 ? kSlots : 32; // producer lanes that issue copies in one round
constexpr int kPage = 16;
constexpr int kD = 128;
constexpr int kPartStride = kD + 4; // floats per (part, head): o[128], m, l, 2 pad (16-byte rows)
// A ring slot holds one page of one kv-head as the two TMA boxes leave it: [dims 0-63 | dims 64-127][K | V][16 tokens][128 B]
constexpr int kQuarterBytes = kPage * 64 * 2;   // 2 KiB: 16 tokens x 64 dims of K (or V)
constexpr int kHalfBytes = 2 * kQuarterBytes;   // 4 KiB: one box = K and V, 64 dims
constexpr int kSlotBytes = 2 * kHalfBytes;      // 8 KiB
constexpr int kRingBytes = kSlots * kSlotBytes; // 96 KiB
constexpr int kMaxGroup = 8;
constexpr int kMaxSeqs = 1024;
constexpr int kCtasPerSm = 8 / kConsumerWarps;
constexpr uint32_t kWaitLimit = 1u << 20; // polls before a wait gives up (about a second at worst)
constexpr int kErrTimeout = 8;
constexpr int kSharedMergeFrom = 9; // a pair cut into this many pieces or more is merged by all five warps of the CTA
constexpr int kMergeWarps = kConsumerWarps + 1; // that arrives last, if the pair ends the CTA's span (consumers + epilogue)
constexpr int kStageBytes = 512 + 16; // per consumer warp: a new K row and V row (256 B each) and their page index
constexpr int kDimGroups = kConsumerThreads / kD; // the pair epilogue maps a consumer thread to one output
static_assert(kConsumerThreads % kD == 0, "dimension and to every kDimGroups-th head of the group");

struct TmaDecodeParams {
    long long page0;            // layer * num_pages: first page of this layer in the tensor map
    const int32_t *block_table; // [rows][table_stride]
    int32_t table_stride, num_pages, max_tokens;
    const int32_t *seq_ids;
    const int32_t *kv_lens;
    int32_t n_seqs, nkvh, group, nh;
    const void *q;
    void *out;
    float *part;
    float scale_log2;
    float *partials;
    int32_t *counters;
    int32_t *error_flag;
    // fused step: row i of k_new / v_new [n_seqs, nkvh, 128] becomes token kv_lens[i] - 1 of sequence i (null: plain decode)
    const char *k_new;
    const char *v_new;
    char *pool_k;                           // K tile of (page 0, kv-head 0) of this layer
    long long page_stride_b, head_stride_b; // bytes between pages / kv-heads
    long long v_offset_b;                   // V tile - K tile of the same (page, kv-head)
    // KV-range split across GPUs (exchange instantiation; out null, part = PeerSink::rows): a pair's finished rows
    // (o, m, l) are written locally like any partial output, and the epilogue warp of the CTA that finished them then
    // stores every value, together with the step number, as one 8-byte word into slot `rank` of EVERY rank's exchange
    // buffer (plain stores into peer memory). The word is its own flag: the reader takes a value once the step beside
    // it is the current one, so no fence, no flag and no count of finished pairs is needed (a system-scope fence costs
    // this GPU about 20 us: two per launch doubled the single-sequence kernel's time).
    PeerSink xchg;
};

constexpr int kMaxXchg = 16; // ranks of one exchange

// The device-side step counter of the exchange: the number of merges completed so far. This launch belongs to the next.
__device__ __forceinline__ uint32_t xchg_step(const TmaDecodeParams &p) {
    return __ldcg(reinterpret_cast<const uint32_t *>(p.xchg.own + p.xchg.epoch_offset)) + 1u;
}

// Exchange mode: n floats of this rank's finished rows, rows[first .. first + n), go -- each with the step beside it, as
// one aligned 8-byte store: value and step arrive together -- into this rank's slot of EVERY rank's buffer. Called by one
// whole warp. Functions of their own on purpose: written into the kernel, the loop over the ranks and its volatile
// stores changed the code of the consumer warps around them, and the exchange instantiation streamed pages 1.8 times
// slower than the ordinary one. Sixteen values are fetched before the first is sent: no load passes a volatile store,
// and one trip to L2 per value would make this the longest step of a short launch.
__device__ __noinline__ void xchg_send_rows(unsigned char *const *table, int world, long long slot_at, const float *rows,
                                            long long first, int n, uint32_t step, int lane) {
    constexpr int kAtOnce = 16;
    for (int i0 = 0; i0 < n; i0 += kAtOnce * 32) {
        float vals[kAtOnce];
#pragma unroll
        for (int u = 0; u < kAtOnce; ++u) {
            const int i = i0 + u * 32 + lane;
            vals[u] = i < n ? __ldcg(rows + first + i) : 0.f;
        }
        for (int pe = 0; pe < world; ++pe) {
            uint2 *dst = reinterpret_cast<uint2 *>(__ldg(reinterpret_cast<const unsigned long long *>(table) + pe)) + slot_at + first;
#pragma unroll
            for (int u = 0; u < kAtOnce; ++u) {
                const int i = i0 + u * 32 + lane;
                if (i < n) {
                    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};\n" ::"l"(dst + i), "r"(__float_as_uint(vals[u])),
                                 "r"(step)
                                 : "memory");
                }
            }
        }
    }
}
// One value (the rows of a sequence without tokens, written by whichever thread owns the dimension).
__device__ __noinline__ void xchg_send_one(unsigned char *const *table, int world, long long at, float v, uint32_t step) {
    for (int pe = 0; pe < world; ++pe) {
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};\n" ::"l"(reinterpret_cast<uint2 *>(__ldg(reinterpret_cast<const unsigned long long *>(table) + pe)) + at),
                     "r"(__float_as_uint(v)), "r"(step)
                     : "memory");
    }
}
// Word index of this rank's slot (of the step's parity) in every rank's buffer.
__device__ __forceinline__ long long xchg_slot_at(const TmaDecodeParams &p, uint32_t step) {
    return ((long long)(step & 1u) * p.xchg.world + p.xchg.rank) * (long long)p.xchg.slot_floats;
}

struct Cursor {
    int s, kvh, j, np, kv_len, remaining;
};

struct Segment {
    int s, kvh, j0, n, kv_len; // pages [j0, j0 + n) of pair (s, kvh): the piece of the pair inside this span
};

// Index arrays passed BY VALUE with the launch (at most kInlineSeqs sequences): for a caller whose arrays are in host
// memory this saves the upload and lets the kernel start before whatever upload precedes it on the stream.
constexpr int kInlineSeqs = 256;
struct InlineIndex {
    int32_t n;                   // 0: the arrays are in device memory (TmaDecodeParams::seq_ids / kv_lens)
    int32_t v[2 * kInlineSeqs];  // seq_ids[n], then kv_lens[n]
};

__device__ __forceinline__ int seq_kv_len(const int32_t *kv_lens, int max_tokens, int s) {
    return min(max(kv_lens[s], 0), max_tokens);
}

__device__ __forceinline__ Segment next_segment(Cursor &c, const int *cum, const TmaDecodeParams &p, const int32_t *kv_lens) {
    Segment sg;
    sg.s = c.s;
    sg.kvh = c.kvh;
    sg.j0 = c.j;
    sg.kv_len = c.kv_len;
    sg.n = min(c.np - c.j, c.remaining);
    c.j += sg.n;
    c.remaining -= sg.n;
    if (c.j == c.np && c.remaining > 0) {
        c.j = 0;
        if (++c.kvh == p.nkvh) {
            c.kvh = 0;
            do { // remaining > 0 guarantees a later sequence with pages; the bound only guards the walk
                ++c.s;
                c.np = cum[c.s + 1] - cum[c.s];
            } while (c.np == 0 && c.s + 1 < p.n_seqs);
            c.kv_len = seq_kv_len(kv_lens, p.max_tokens, c.s);
        }
    }
    return sg;
}

// Polls a barrier phase; gives up after kWaitLimit polls or when another warp of the CTA already gave up.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((i & 1023u) == 1023u && *abort_flag != 0) {
            return false;
        }
    }
    return false;
}

// kXchg: the exchange mode of a KV-range split (PeerSink) -- a separate instantiation, so that the ordinary decode
// kernel carries none of its code (with a run-time switch the peer stores, although never executed, cost the ordinary
// kernel 2 us of 47). The two differ in the epilogue warp only: in exchange mode it is handed every pair, whole ones
// too, and sends the rows out (xchg_send_rows); the consumer warps run the same code in both.
// kShare: launches with few pairs for their grid, whose pairs can be in many pieces, carry the shared merge (all five
// warps of the last-arriving CTA); the others do not even contain its code -- this kernel's timing moves by a
// microsecond with what is compiled around its hot loop.
template <bool kBf16, bool kXchg, bool kShare>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
    paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ InlineIndex ix,
                            TmaDecodeParams p) {
    extern __shared__ unsigned char smem_raw[];
    // the 128-byte swizzle is a function of the shared-memory address: slots must start on 1 KiB boundaries
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t ring_u32 = (raw_u32 + 1023u) & ~1023u;
    unsigned char *aligned = smem_raw + (ring_u32 - raw_u32);
    float *red_o = reinterpret_cast<float *>(aligned + kRingBytes);                       // [warps][group][kD]
    float *red_ml = red_o + kConsumerWarps * p.group * kD;                                // [warps][kMaxGroup][2]
    uint64_t *bars = reinterpret_cast<uint64_t *>(red_ml + kConsumerWarps * kMaxGroup * 2); // full[], empty[], epi_ready, epi_done, verdict
    int *cum = reinterpret_cast<int *>(bars + 2 * kSlots + 3);                                // [n_seqs + 1]
    int *rows = cum + p.n_seqs + 1;                                                           // [n_seqs] block-table rows
    // new-row staging, 16-byte aligned, one block per consumer warp
    const uint32_t stage_u32 = (smem_u32(rows + p.n_seqs) + 15u) & ~15u;
    __shared__ int s_abort;
    __shared__ int s_verdict; // shared merge: 1 = this CTA arrived last at its final pair and every warp takes a share
    const uint32_t bars_u32 = smem_u32(bars);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int32_t *seq_ids = ix.n > 0 ? ix.v : p.seq_ids;
    const int32_t *kv_lens = ix.n > 0 ? ix.v + ix.n : p.kv_lens;

    if (tid == 0) {
        for (int i = 0; i < 2 * kSlots; ++i) {
            mbar_init(bars_u32 + i * 8, 1);
        }
        mbar_init(bars_u32 + 2 * kSlots * 8, kConsumerThreads); // epi_ready: every consumer thread arrives
        mbar_init(bars_u32 + (2 * kSlots + 1) * 8, 1);          // epi_done: the epilogue warp's lane 0
        mbar_init(bars_u32 + (2 * kSlots + 2) * 8, 1);          // verdict: the epilogue warp's lane 0, once
        s_abort = 0;
        mbar_init_fence();
    }
    // -- page counts and block-table rows of all sequences: ONE round trip to global memory by all threads, then the
    //    prefix sums (warp 0, in place) --------------------------------------------------------------------------
    for (int s = tid; s < p.n_seqs; s += kThreads) {
        cum[s + 1] = (seq_kv_len(kv_lens, p.max_tokens, s) + kPage - 1) / kPage;
        rows[s] = seq_ids ? seq_ids[s] : s;
    }
    if (warp == kProducerWarp && lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tmap)) : "memory");
    }
    __syncthreads();
    if (warp == 0) {
        int running = 0;
        if (lane == 0) {
            cum[0] = 0;
        }
        for (int base = 0; base < p.n_seqs; base += 32) {
            const int s = base + lane;
            int incl = s < p.n_seqs ? cum[s + 1] : 0;
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

    const bool partial = p.part != nullptr; // (exchange mode: the rows on their way out, PeerSink::rows)
    // -- sequences without any token: the output row is zero (partial: o = 0, m = -inf, l = 0). Called by threads
    //    0..127 at least, after their grid_dependency_wait.
    auto write_empty_pairs = [&]() {
        const uint32_t step = kXchg ? xchg_step(p) : 0u;
        for (int pair = blockIdx.x; pair < n_pairs; pair += gridDim.x) {
            const int s = pair / p.nkvh, kvh = pair - s * p.nkvh;
            if (cum[s + 1] - cum[s] != 0) {
                continue;
            }
            if (tid >= kD) {
                continue;
            }
            for (int h = 0; h < p.group; ++h) {
                const long long row = (long long)s * p.nh + kvh * p.group + h;
                if constexpr (kXchg) {
                    const long long at = xchg_slot_at(p, step) + row * (kD + 2);
                    xchg_send_one(p.xchg.table, p.xchg.world, at + tid, 0.f, step);
                    if (tid == 0) {
                        xchg_send_one(p.xchg.table, p.xchg.world, at + kD, -INFINITY, step);
                        xchg_send_one(p.xchg.table, p.xchg.world, at + kD + 1, 0.f, step);
                    }
                } else if (partial) {
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
    };
    if (x0 >= x1) {
        grid_dependency_wait(); // outputs may still be in use by the previous kernel on the stream
        write_empty_pairs();
        return; // exiting counts as this CTA's launch_dependents
    }

    // -- first page of the span ----------------------------------------------------------------------------
    Cursor cur;
    {
        int lo = 0, hi = p.n_seqs - 1;
        while (lo < hi) { // last s with cum[s] * nkvh <= x0; it owns page x0 and is never an empty sequence
            const int mid = (lo + hi + 1) >> 1;
            if ((long long)cum[mid] * p.nkvh <= x0) {
                lo = mid;
            } else {
                hi = mid - 1;
            }
        }
        cur.s = lo;
        cur.np = cum[lo + 1] - cum[lo];
        const int r = int(x0 - (long long)cum[lo] * p.nkvh);
        cur.kvh = r / cur.np;
        cur.j = r - cur.kvh * cur.np;
        cur.kv_len = seq_kv_len(kv_lens, p.max_tokens, lo);
        cur.remaining = int(x1 - x0);
    }

    // ======================================= producer warp ================================================
    if (warp == kProducerWarp) {
        int n = 0; // pages issued so far; page n uses slot n % kSlots for the (n / kSlots)-th time
        bool dead = false, waited = false;
        while (cur.remaining > 0 && !dead) {
            const Segment sg = next_segment(cur, cum, p, kv_lens);
            if (sg.n <= 0) {
                break; // inconsistent lengths: the consumers flag it
            }
            const long long tbase = (long long)rows[sg.s] * p.table_stride + sg.j0;
            // first page the kernel before this one on the stream may still be writing: the one holding token kv_len - 2
            const int guard_page = (max(sg.kv_len, 2) - 2) / kPage;
            for (int base = 0; base < sg.n && !dead; base += kIssueLanes) {
                // One page per lane: kIssueLanes lanes fetch their table entries in one coalesced read and each lane
                // issues the copies of its own page, so the per-instruction latency of TMA issue is paid once
                // per 32 pages instead of once per page. A lane whose slot is still in use spins on that slot's
                // "empty" barrier; the lanes ahead of it have already issued, and the consumers free slots in
                // page order, so every wait ends. No more lanes than ring slots take part in a round: two lanes
                // on one slot would wait for consecutive phases of the same barrier, and a parity wait cannot tell
                // phase k + 1 from phase k - 1.
                if (!waited && sg.j0 + min(base + kIssueLanes, sg.n) > guard_page) {
                    // these copies reach the sequence's newest rows, which may come from the previous kernel on the
                    // stream (everything before it was there long ago)
                    grid_dependency_wait();
                    waited = true;
                }
                const bool active = lane < kIssueLanes && base + lane < sg.n;
                int ok = 1;
                if (active) {
                    int page = p.block_table[tbase + base + lane];
                    if (page < 0 || page >= p.num_pages) {
                        atomicOr(p.error_flag, kErrBadPage);
                        page = 0;
                    }
                    const int mine = n + lane;
                    const int slot = mine % kSlots, use = mine / kSlots;
                    const uint32_t full_bar = bars_u32 + slot * 8, empty_bar = bars_u32 + (kSlots + slot) * 8;
                    if (use > 0 && !wait_or_abort(empty_bar, uint32_t(use - 1) & 1u, &s_abort)) {
                        ok = 0;
                    } else {
                        mbar_arrive_expect_tx(full_bar, kSlotBytes);
                        const int c3 = int((p.page0 + page) * 2); // (page, K) ; the box also takes (page, V)
                        const uint32_t dst = ring_u32 + slot * kSlotBytes;
                        tma_load_4d(dst, &tmap, 0, 0, sg.kvh, c3, full_bar);
                        tma_load_4d(dst + kHalfBytes, &tmap, 64, 0, sg.kvh, c3, full_bar);
                    }
                }
                if (__any_sync(0xffffffffu, ok == 0)) {
                    dead = true;
                    break;
                }
                n += min(kIssueLanes, sg.n - base);
            }
        }
        if (dead && lane == 0) {
            s_abort = 1;
            atomicOr(p.error_flag, kErrTimeout);
            // wait (bounded) for the copies this warp still has in flight before the CTA may exit
            for (int back = 1; back <= kSlots && back <= n; ++back) {
                const int m = n - back;
                mbar_wait_bounded(bars_u32 + (m % kSlots) * 8, uint32_t(m / kSlots) & 1u, kWaitLimit);
            }
        }
        return;
    }

    // ======================================= epilogue warp ================================================
    // Walks the same segments as everyone else. For a pair that is cut across CTAs it waits until the consumers
    // have written this CTA's partial, publishes it (fence + arrival count) and, if this was the last arrival,
    // merges all partials of the pair -- off the consumers' critical path, so the ring keeps draining meanwhile.
    const uint32_t epi_ready = bars_u32 + 2 * kSlots * 8, epi_done = bars_u32 + (2 * kSlots + 1) * 8;
    const uint32_t verdict_bar = bars_u32 + (2 * kSlots + 2) * 8;
    // The shared merge keeps its warps' unfinished states in this CTA's own five slots behind the partial results.
    float *stash = p.partials + ((long long)gridDim.x + n_pairs + (long long)blockIdx.x * kMergeWarps) * p.group * kPartStride;
    if (warp == kEpilogueWarp) {
        grid_dependency_wait(); // counters and partials are shared with the previous launch
        const uint32_t step = kXchg ? xchg_step(p) : 0u;
        int k = 0; // cut segments handled so far
        while (cur.remaining > 0) {
            const Segment sg = next_segment(cur, cum, p, kv_lens);
            if (sg.n <= 0) {
                break;
            }
            const int pair = sg.s * p.nkvh + sg.kvh;
            const int pair_np = cum[sg.s + 1] - cum[sg.s];
            const long long pair_off = (long long)cum[sg.s] * p.nkvh + (long long)sg.kvh * pair_np;
            const int c_first = int(pair_off / span), c_last = int((pair_off + pair_np - 1) / span);
            const int expected = c_last - c_first + 1;
            if (expected == 1 && !kXchg) {
                continue; // the consumers wrote the final output themselves
            }
            if (!wait_or_abort(epi_ready, uint32_t(k) & 1u, &s_abort)) {
                if (lane == 0) {
                    s_abort = 1;
                    atomicOr(p.error_flag, kErrTimeout);
                }
                break;
            }
            const long long row0 = (long long)sg.s * p.nh + sg.kvh * p.group;
            if (kXchg && expected == 1) { // the consumers have completed the pair's rows: off they go
                xchg_send_rows(p.xchg.table, p.xchg.world, xchg_slot_at(p, step), p.part, row0 * (kD + 2), p.group * (kD + 2),
                               step, lane);
                if (lane == 0) {
                    mbar_arrive(epi_done);
                }
                ++k;
                continue;
            }
            int last = 0;
            if (lane == 0) {
                // One read-modify-write that is both the release of this CTA's partial (the consumers' stores are ordered
                // before it by the mbarrier; release is cumulative) and the acquire of the other CTAs' partials: half a
                // microsecond less on every launch's tail than a fence on either side of a relaxed atomic.
                int old;
                asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;\n" : "=r"(old) : "l"(p.counters + pair) : "memory");
                last = (old == expected - 1) ? 1 : 0;
            }
            __syncwarp(); // the other lanes' reads below come after lane 0's acquire
            last = __shfl_sync(0xffffffffu, last, 0);
            // A pair in many pieces is merged in five shares (share w = parts w, w + 5, ...) whose unfinished states are
            // then folded: by all five warps of the CTA where the pair ends the CTA's span (the consumers have nothing
            // left to do and wait for the verdict), by this warp alone, share after share, where the consumers are still
            // streaming. The arithmetic and its order are the same either way: the bits do not depend on who arrived last.
            const bool shared_merge = kShare && expected >= kSharedMergeFrom;
            const bool helpers = shared_merge && cur.remaining == 0;
            if (helpers && lane == 0) {
                s_verdict = last;
                mbar_arrive(verdict_bar); // release: the consumers read s_verdict after their wait
            }
            if (last) {
                const float *first = p.partials + (long long)(c_first + pair) * p.group * kPartStride;
                if constexpr (kShare) {
                  if (shared_merge) {
                    if (helpers) {
                        warp_merge_share<kBf16>(first, expected, kConsumerWarps, kMergeWarps, p.group, lane, stash);
                        named_barrier_sync(2, kMergeWarps * 32); // every share is stashed; all parts have been read
                    } else {
                        for (int w = 0; w < kMergeWarps; ++w) {
                            warp_merge_share<kBf16>(first, expected, w, kMergeWarps, p.group, lane, stash);
                        }
                        __syncwarp();
                    }
                    warp_merge_finish<kBf16>(stash, kMergeWarps, p.group, lane, p.out, p.part, row0);
                  }
                }
                if (!shared_merge) {
                    warp_combine_partials<kBf16>(first, expected, p.group, lane, p.out, p.part, row0);
                }
                if constexpr (kXchg) {
                    __syncwarp(); // the lanes' stores of the merged rows come before the loads that send them
                    xchg_send_rows(p.xchg.table, p.xchg.world, xchg_slot_at(p, step), p.part, row0 * (kD + 2),
                                   p.group * (kD + 2), step, lane);
                }
                if (lane == 0) {
                    p.counters[pair] = 0; // ready for the next launch
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(epi_done);
            }
            ++k;
        }
        return;
    }

    // ======================================= consumer warps ===============================================
    const int g = lane >> 2, q4 = lane & 3; // MMA fragment coordinates: row group, column pair
    // ldmatrix row addresses. A tile is [half (64 dims)][16 tokens][128 B] with chunk' = chunk ^ (token % 8):
    //   K (not transposed): lane supplies token lm_r + 8 * (mi & 1), chunk 2 * ks + (mi >> 1)
    //   V (transposed):     lane supplies token lm_r + 8 * (mi >> 1), chunk 2 * mt + (mi & 1)
    const int lm_r = lane & 7, lm_mi = lane >> 3;
    const int k_tok = lm_r + 8 * (lm_mi & 1), k_cc0 = lm_mi >> 1;
    const int v_tok = lm_r + 8 * (lm_mi >> 1), v_cc0 = lm_mi & 1;

    // q, the newest K/V rows and every output belong to the stream's order: nothing of them is touched before the
    // previous kernel has completed. (The ring is already filling: the producer copies older pages meanwhile.)
    grid_dependency_wait();
    // Only now may the successor on the stream be scheduled: whatever starts early behind this grid can then rely on
    // everything BEFORE this grid's predecessor being complete (see the overlap contract in paged_kv.h).
    grid_launch_dependents();
    write_empty_pairs();
    float m2[2], l[2], o_acc[8][4];
    uint32_t qf[8][2];
    auto reset_state = [&]() {
        m2[0] = m2[1] = -INFINITY;
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            o_acc[mt][0] = o_acc[mt][1] = o_acc[mt][2] = o_acc[mt][3] = 0.f;
        }
    };
    reset_state();

    int n_base = 0, n_cut = 0; // pages consumed so far; cut segments handed to the epilogue warp so far
    bool dead = false;
    while (cur.remaining > 0) {
        const Segment sg = next_segment(cur, cum, p, kv_lens);
        if (sg.n <= 0) { // cannot happen with consistent lengths; leave rather than spin (uniform over the CTA)
            if (tid == 0) {
                atomicOr(p.error_flag, kErrBadSeq);
            }
            break;
        }
        {
            // query fragments of this pair: B operand [k = dim][n = head], head g of the group (zero beyond it)
            const uint32_t *q_row = reinterpret_cast<const uint32_t *>(
                static_cast<const char *>(p.q) + ((long long)sg.s * p.nh + sg.kvh * p.group + g) * (kD * 2));
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qf[ks][0] = g < p.group ? q_row[ks * 8 + q4] : 0u;
                qf[ks][1] = g < p.group ? q_row[ks * 8 + 4 + q4] : 0u;
            }
        }
        // fused step: index in this segment of the pair's last page, which receives the new row; the warp that will
        // take that page fetches the row (K: lanes 0-15, V: lanes 16-31, 16 bytes each) and the page index now
        const int new_i = p.k_new != nullptr ? (cum[sg.s + 1] - cum[sg.s]) - 1 - sg.j0 : -1;
        const bool brings_new = new_i >= 0 && new_i < sg.n && new_i % kConsumerWarps == warp;
        const uint32_t my_stage = stage_u32 + warp * kStageBytes;
        if (brings_new) {
            const char *src = (lane < 16 ? p.k_new : p.v_new) + ((long long)sg.s * p.nkvh + sg.kvh) * (kD * 2) + (lane & 15) * 16;
            cp_async_16(my_stage + lane * 16, src, 16);
            if (lane == 0) {
                const int32_t *entry = p.block_table + (long long)rows[sg.s] * p.table_stride + sg.j0 + new_i;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(my_stage + 512), "l"(entry) : "memory");
            }
            cp_async_commit();
        }

        for (int i = warp; i < sg.n && !dead; i += kConsumerWarps) {
            const int n = n_base + i;
            const int slot = n % kSlots, use = n / kSlots;
            const uint32_t full_bar = bars_u32 + slot * 8, empty_bar = bars_u32 + (kSlots + slot) * 8;
            if (!wait_or_abort(full_bar, uint32_t(use) & 1u, &s_abort)) {
                dead = true;
                if (lane == 0) {
                    s_abort = 1;
                    atomicOr(p.error_flag, kErrTimeout);
                }
                break;
            }
            const uint32_t tile = ring_u32 + slot * kSlotBytes;
            const int n_valid = min(kPage, sg.kv_len - (sg.j0 + i) * kPage);
            const bool patch = brings_new && i == new_i;
            if (patch) {
                // the new row: over slot n_valid - 1 of the tile (swizzled like the TMA copy) and into the page itself
                cp_async_wait<0>();
                __syncwarp();
                const int r = n_valid - 1, cc = lane & 15;
                uint32_t w0, w1, w2, w3;
                int page;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                             : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                             : "r"(my_stage + lane * 16));
                asm volatile("ld.shared.s32 %0, [%1];\n" : "=r"(page) : "r"(my_stage + 512));
                const uint32_t a = tile + (lane < 16 ? 0 : kQuarterBytes) + (cc >> 3) * kHalfBytes + r * 128 +
                                   (((cc & 7) ^ (r & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(a), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                if (page >= 0 && page < p.num_pages) { // (the producer has flagged a bad entry already)
                    char *dst = p.pool_k + (long long)page * p.page_stride_b + (long long)sg.kvh * p.head_stride_b +
                                (lane < 16 ? 0 : p.v_offset_b) + r * (kD * 2) + cc * 16;
                    *reinterpret_cast<uint4 *>(dst) = make_uint4(w0, w1, w2, w3);
                }
                __syncwarp();
            }
            if (n_valid < kPage) {
                // Rows past the sequence's end hold whatever the page held before. K rows are neutralised by the
                // score mask; V rows are cleared here so that 0 * garbage cannot make a NaN.
                const int chunks = (kPage - n_valid) * 16;
                for (int c = lane; c < chunks; c += 32) {
                    const int r = n_valid + (c >> 4), cc = c & 15;
                    const uint32_t a = tile + kQuarterBytes + (cc >> 3) * kHalfBytes + r * 128 + ((cc & 7) << 4);
                    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(a), "r"(0u) : "memory");
                }
                __syncwarp();
            }
            // S^T = K . Q^T
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t k_row = tile + k_tok * 128;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, k_row + (ks >> 2) * kHalfBytes + ((((2 * ks + k_cc0) & 7) ^ lm_r) << 4));
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
            const uint32_t v_row = tile + kQuarterBytes + v_tok * 128;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, v_row + (mt >> 2) * kHalfBytes + ((((2 * mt + v_cc0) & 7) ^ lm_r) << 4));
                mma_16816<kBf16>(o_acc[mt], a, b0, b1);
            }
            // hand the slot back: every lane's reads are done once the warp has converged here
            if (n_valid < kPage || patch) {
                fence_proxy_async_smem(); // the cleared / new rows were ordinary stores; the next writer is the TMA unit
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(empty_bar);
            }
        }
        n_base += sg.n;

        // -- the pair (or this span's piece of it) is done: merge the consumer warps, then publish --------------
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
        named_barrier_sync(1, kConsumerThreads);

        const int pair = sg.s * p.nkvh + sg.kvh;
        const int pair_np = cum[sg.s + 1] - cum[sg.s];
        const long long pair_off = (long long)cum[sg.s] * p.nkvh + (long long)sg.kvh * pair_np;
        const int c_first = int(pair_off / span), c_last = int((pair_off + pair_np - 1) / span);
        const int expected = c_last - c_first + 1;
        float *slot_out = p.partials + (long long)(blockIdx.x + pair) * p.group * kPartStride;

        // consumer thread `tid` owns output dimension tid % 128 of the heads h = tid / 128 (mod kDimGroups); the
        // heads are independent chains of shared-memory reads, unrolled so that they overlap
        const int dim = tid & (kD - 1);
        const long long row0 = (long long)sg.s * p.nh + sg.kvh * p.group;
#pragma unroll
        for (int hh = 0; hh < kMaxGroup / kDimGroups; ++hh) {
            const int h = hh * kDimGroups + tid / kD;
            if (h >= p.group) {
                continue;
            }
            float mw[kConsumerWarps], m_all = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                mw[w] = red_ml[(w * kMaxGroup + h) * 2];
                m_all = fmaxf(m_all, mw[w]);
            }
            float l_all = 0.f, o = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                const float wgt = mw[w] == -INFINITY ? 0.f : fast_exp2(mw[w] - m_all);
                l_all = fmaf(red_ml[(w * kMaxGroup + h) * 2 + 1], wgt, l_all);
                o = fmaf(red_o[(w * p.group + h) * kD + dim], wgt, o);
            }
            if (expected == 1) {
                const long long row = row0 + h;
                const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
                if (partial) {
                    p.part[row * (kD + 2) + dim] = o * inv;
                    if (dim == 0) {
                        p.part[row * (kD + 2) + kD] = m_all * 0.6931471805599453f; // log2 units -> natural log
                        p.part[row * (kD + 2) + kD + 1] = l_all;
                    }
                } else {
                    store_out<kBf16>(p.out, row * kD + dim, o * inv);
                }
            } else {
                slot_out[h * kPartStride + dim] = o; // un-normalised, relative to m_all
                if (dim == 0) {
                    slot_out[h * kPartStride + kD] = m_all;
                    slot_out[h * kPartStride + kD + 1] = l_all;
                }
            }
        }

        if (expected > 1 || kXchg) {
            // Hand the pair to the epilogue warp and carry on with the next pages (exchange mode: whole pairs too --
            // that warp sends their rows to the other ranks). It must have finished the
            // previous cut pair first (the two barriers advance one phase per pair); that wait is normally over
            // long before, since a merge takes microseconds and a segment tens of them.
            if (n_cut > 0 && !dead && !wait_or_abort(epi_done, uint32_t(n_cut - 1) & 1u, &s_abort)) {
                dead = true;
                if (lane == 0) {
                    s_abort = 1;
                    atomicOr(p.error_flag, kErrTimeout);
                }
            }
            mbar_arrive(epi_ready); // release: this thread's partial stores are ordered before the epilogue's fence
            ++n_cut;
        }
        reset_state();
        // red_o / red_ml are next written after this pair's readers have passed the barrier below
        named_barrier_sync(1, kConsumerThreads);
        if (kShare && cur.remaining == 0 && expected >= kSharedMergeFrom && !dead) {
            // the span ended inside a pair in many pieces: if this CTA is the one that merges it (the epilogue warp says),
            // take a share of the parts -- warp w folds parts w, w + 5, ... -- and meet the others
            if (wait_or_abort(verdict_bar, 0u, &s_abort) && s_verdict != 0) {
                const float *first = p.partials + (long long)(c_first + pair) * p.group * kPartStride;
                warp_merge_share<kBf16>(first, expected, warp, kMergeWarps, p.group, lane, stash);
                named_barrier_sync(2, kMergeWarps * 32);
            }
        }
    }
}

// ---- host side --------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
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

size_t smem_bytes(int group, int n_seqs) {
    return 1024 + size_t(kRingBytes) + size_t(kConsumerWarps) * group * kD * sizeof(float) +
           size_t(kConsumerWarps) * kMaxGroup * 2 * sizeof(float) + (2 * kSlots + 3) * sizeof(uint64_t) +
           size_t(2 * n_seqs + 1) * sizeof(int) + 16 + size_t(kConsumerWarps) * kStageBytes;
}

template <bool kBf16, bool kXchg, bool kShare>
void launch(cudaStream_t s, const CUtensorMap &tmap, const InlineIndex &ix, const TmaDecodeParams &p, int grid, size_t smem,
            bool overlap) {
    static std::once_flag once[64];
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    std::call_once(once[dev & 63], [dev] {
        int optin = 0;
        LLAISYS_CUDA_CHECK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        cudaFuncAttributes attr{};
        LLAISYS_CUDA_CHECK(cudaFuncGetAttributes(&attr, paged_decode_tma_kernel<kBf16, kXchg, kShare>));
        LLAISYS_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_tma_kernel<kBf16, kXchg, kShare>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                optin - int(attr.sharedSizeBytes)));
    });
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(unsigned(kThreads));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = overlap ? 1 : 0;
    LLAISYS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, paged_decode_tma_kernel<kBf16, kXchg, kShare>, tmap, ix, p));
}

} // namespace

int make_kv_tensor_map(void *out_128_bytes, void *pool_base, uint64_t total_rows, uint32_t total_rows_per_head_block,
                       llaisysDataType_t dtype) {
    if (dtype != LLAISYS_DTYPE_BF16 && dtype != LLAISYS_DTYPE_F16) {
        return -1;
    }
    // rows are addressed with 32-bit coordinates; the base must satisfy the TMA's 16-byte rule
    if (total_rows == 0 || total_rows_per_head_block == 0 || total_rows % (uint64_t(kPage) * total_rows_per_head_block) != 0 ||
        total_rows >= (uint64_t(1) << 31) || reinterpret_cast<uintptr_t>(pool_base) % 16 != 0) {
        return -1;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) {
        return -1;
    }
    // The pool as a 4-D tensor: [page-and-K|V][kv-head][slot 0..15][128 elements]. One box = 64 elements x 16
    // slots x 1 head x 2 (K and V of the page): two 2 KiB blocks in shared memory, each with the 128-byte swizzle
    // (16-byte chunks permuted by slot % 8).
    const cuuint64_t n_heads = total_rows_per_head_block;
    const cuuint64_t dims[4] = {cuuint64_t(kD), cuuint64_t(kPage), n_heads, cuuint64_t(total_rows / (kPage * n_heads))};
    const cuuint64_t strides[3] = {cuuint64_t(kD * 2), cuuint64_t(kPage * kD * 2), cuuint64_t(kPage * kD * 2) * n_heads};
    const cuuint32_t box[4] = {64, cuuint32_t(kPage), 1, 2};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    CUtensorMap map;
    const CUresult rc =
        encode(&map, dtype == LLAISYS_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
               pool_base, dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        return -1;
    }
    static_assert(sizeof(CUtensorMap) == 128, "tensor map blob size");
    memcpy(out_128_bytes, &map, sizeof(map));
    return 0;
}

int attention_decode_tma(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                         const void *q, float scale, const AttnOut &out, const AttnScratch &scratch, const void *k_new,
                         const void *v_new, const char **why) {
    const char *dummy = nullptr;
    const char *&reason = why != nullptr ? *why : dummy;
    const bool bf16 = dtype == LLAISYS_DTYPE_BF16;
    if (!(bf16 || dtype == LLAISYS_DTYPE_F16) || kv.d != kD || kv.page_size != kPage || kv.nkvh <= 0 ||
        batch.nh % kv.nkvh != 0 || batch.nh / kv.nkvh > kMaxGroup || batch.q_starts != nullptr || batch.const_q_len != 1) {
        reason = "needs 16-bit K/V, head_dim 128, 16-token pages, at most 8 query heads per kv head, one query per sequence";
        return -1;
    }
    const bool inline_index = batch.host_seq_ids != nullptr && batch.host_kv_lens != nullptr && batch.n_seqs <= kInlineSeqs;
    if (kv.tma_desc == nullptr || kv.block_table == nullptr || (batch.kv_lens == nullptr && !inline_index)) {
        reason = "the pool carries no tensor map (the driver could not encode one), or block table / lengths are missing";
        return -1;
    }
    if (batch.n_seqs <= 0 || batch.n_seqs > kMaxSeqs) {
        reason = "more than 1024 sequences in one call: split the batch";
        return -1;
    }
    if (reinterpret_cast<uintptr_t>(q) % 4 != 0) {
        reason = "q is not 4-byte aligned";
        return -1;
    }
    if ((k_new == nullptr) != (v_new == nullptr) || reinterpret_cast<uintptr_t>(k_new) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(v_new) % 16 != 0) {
        reason = "the new K/V rows of a fused step must both be given and be 16-byte aligned";
        return -1;
    }
    const int group = batch.nh / kv.nkvh;
    const int grid = decode_grid_size(batch.n_seqs, kv.nkvh, batch.max_kv_len);
    const size_t n_pairs = size_t(batch.n_seqs) * kv.nkvh;
    if (scratch.partials == nullptr || scratch.counters == nullptr || scratch.error_flag == nullptr ||
        scratch.partials_floats < (size_t(grid) * (1 + kMergeWarps) + n_pairs) * group * kPartStride ||
        scratch.counters_len < n_pairs) {
        reason = "split-KV scratch missing or too small for this batch";
        return -1;
    }
    if (out.peers != nullptr) {
        const PeerSink &x = *out.peers;
        if (out.out != nullptr || out.part != nullptr || x.table == nullptr || x.own == nullptr || x.rows == nullptr || x.world < 1 || x.world > kMaxXchg || x.rank < 0 || x.rank >= x.world ||
            size_t(batch.n_seqs) * batch.nh * (kD + 2) > x.slot_floats) {
            reason = "exchange slots: bad rank / world size, rows do not fit a slot, or another output was given too";
            return -1;
        }
    } else if ((out.out != nullptr) == (out.part != nullptr)) {
        reason = "exactly one of out and part must be given";
        return -1;
    }
    TmaDecodeParams p;
    p.page0 = kv.tma_page0;
    p.block_table = kv.block_table;
    p.table_stride = kv.table_stride;
    p.num_pages = kv.num_pages;
    p.max_tokens = kv.table_stride * kPage;
    p.seq_ids = batch.seq_ids;
    p.kv_lens = batch.kv_lens;
    p.n_seqs = batch.n_seqs;
    p.nkvh = kv.nkvh;
    p.group = group;
    p.nh = batch.nh;
    p.q = q;
    p.out = out.out;
    p.part = out.peers != nullptr ? out.peers->rows : out.part;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.partials = scratch.partials;
    p.counters = scratch.counters;
    p.error_flag = scratch.error_flag;
    p.k_new = static_cast<const char *>(k_new);
    p.v_new = static_cast<const char *>(v_new);
    p.pool_k = static_cast<char *>(kv.k_base);
    p.page_stride_b = kv.page_stride * 2;
    p.head_stride_b = kv.head_stride * 2;
    p.v_offset_b = static_cast<char *>(kv.v_base) - static_cast<char *>(kv.k_base);
    p.xchg = PeerSink{};
    if (out.peers != nullptr) {
        p.xchg = *out.peers;
    }
    CUtensorMap tmap;
    memcpy(&tmap, kv.tma_desc, sizeof(tmap));
    const size_t smem = smem_bytes(group, batch.n_seqs);
    auto s = static_cast<cudaStream_t>(stream);
    static thread_local InlineIndex ix; // 2 KB: kept off the stack, filled only when the caller has host arrays
    ix.n = 0;
    if (batch.host_seq_ids != nullptr && batch.host_kv_lens != nullptr && batch.n_seqs <= kInlineSeqs) {
        ix.n = batch.n_seqs;
        memcpy(ix.v, batch.host_seq_ids, size_t(batch.n_seqs) * sizeof(int32_t));
        memcpy(ix.v + batch.n_seqs, batch.host_kv_lens, size_t(batch.n_seqs) * sizeof(int32_t));
    }
    const bool xchg = out.peers != nullptr;
    // pairs can be in kSharedMergeFrom pieces or more only where the grid has that many CTAs per pair
    const bool share = size_t(grid) >= n_pairs * size_t(kSharedMergeFrom - 1);
    auto go = [&](auto bf, auto xc, auto sh) {
        launch<decltype(bf)::value, decltype(xc)::value, decltype(sh)::value>(s, tmap, ix, p, grid, smem, kv.overlap_launch);
    };
    auto pick_share = [&](auto bf, auto xc) {
        share ? go(bf, xc, std::true_type{}) : go(bf, xc, std::false_type{});
    };
    auto pick_xchg = [&](auto bf) { xchg ? pick_share(bf, std::true_type{}) : pick_share(bf, std::false_type{}); };
    bf16 ? pick_xchg(std::true_type{}) : pick_xchg(std::false_type{});
    check_launch("paged_decode_tma");
    return 0;
}

} // namespace llaisys::kernels
