// K4: chunked-prefill attention over the page pool on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Roofline: tensor. Algorithmic flops per sequence = 4 * nh * d * sum over chunk rows of visible keys
//                                                  = 4 * nh * 128 * (L * C + L * (L + 1) / 2)
// for a chunk of L queries after C cached tokens (QK^T and PV, 2 flops per multiply-add; masked work not counted).
//
// Work: a TILE is (sequence, block of 128 chunk rows, query head); it visits its visible keys 64 at a time (a BLOCK:
// 4 pages). All blocks of all tiles, in the order (sequence, row block, head, key block), form one line that is cut
// into equal pieces, one per CTA of a fixed grid of 2 x SMs -- so every CTA gets the same number of blocks whatever
// the mix of sequence lengths (a one-CTA-per-tile grid ran configuration 3's 384 tiles of 13..96 blocks on 296 CTA
// slots and took the time of its longest tile; one 65536-token sequence with a 512-token chunk -- 48 tiles -- used a
// sixth of the GPU and took 1075 us where this grid takes 233). A piece covers the end of one
// tile, whole tiles, and the beginning of another: each such FRAGMENT is run like a tile. A fragment that is its whole
// tile normalises and stores its rows; otherwise it stores the unnormalised accumulator and the rows' (max, sum) into
// a per-CTA slot of a workspace and counts itself in; the fragment that arrives last for its tile merges the others
// with the accumulator it still holds in tensor memory (summing in the order of the CTAs, not of arrival: the bits do
// not depend on who was last) and stores the rows. Nobody waits for anybody. When there are
// few blocks the pieces are kept long enough that merging stays cheaper than the blocks it saves, and CTAs past the
// last piece exit at once.
//
// Per CTA: 128 query rows in shared memory per fragment; K/V arrive 64 tokens at a time:
//   warp 4 (producer)  reads the block table (32 entries at a time, a group ahead of use) and issues TMA tiles
//                      (16 tokens x 64 dims, 128-byte swizzle) into a two-stage K/V ring -- K as [2 dim-halves][64 tokens][128 B], V the same -- running ahead
//                      across fragment boundaries;
//   warp 5 (MMA)       one thread issues tcgen05.mma (M 128, K 16, bf16/f16 -> f32):
//                        S = Q . K^T      N 64, 8 instructions, both operands K-major, accumulator S[buf] in TMEM
//                        O += P . V       N 128, 4 instructions, P from TMEM (A operand), V MN-major (the page layout
//                                         keeps head_dim contiguous), accumulator O in TMEM
//                      QK^T of block i+1 is issued before PV of block i, so the tensor pipe works under the softmax;
//   warps 0-3          the 128 softmax threads, one query row each (TMEM lane = row): tcgen05.ld S, causal mask,
//                      running max / sum in the log2 domain, P = 2^(s - m) as packed 16-bit pairs written over the
//                      first 32 columns of the S buffer they came from, O rescaled in TMEM only when a row's max grew
//                      by more than 2^8 since the last rescale (the stale max is used consistently for P and the
//                      sum). After a fragment's last block they also load the next fragment's Q rows.
// TMEM: 256 columns per CTA: S double-buffered (2 x 64) + O (128). Shared memory: Q 32 KiB + K/V 2 x 32 KiB = 96 KiB,
// so TWO CTAs share an SM (and its 512 TMEM columns): while one CTA's 128 softmax threads work on a block, the other
// CTA's MMAs keep the tensor pipe busy.
// What bounds a block (measured with clock64 stamps per role): the thread that issues the MMAs. tcgen05.mma issue keeps
// pace with execution (8 QK^T instructions take the 300 to 600 clocks the pipe needs for them), so every wait, commit
// and loop step of that thread is time the pipe idles; a block costs it about 1100 clocks of MMAs and as much again
// around them. Hence one commit per batch of MMAs and no barrier that another already implies.
//
// Synchronisation is mbarriers only (plus one named barrier among the softmax threads around the arrival count);
// tcgen05.commit arrives on them when the tensor pipe has finished. Barrier phases run on across fragments: stage and
// parity come from the count of blocks the CTA has done. Every wait is bounded: a wait that runs out sets bit 8 of the
// error word and the CTA winds down (TMEM is freed, arrival counts stay consistent) instead of hanging.
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
constexpr int kBlockM = 128;                 // query rows per tile
constexpr int kBlockN = 64;                  // keys per K/V block (4 pages)
constexpr int kPagesPerBlock = kBlockN / kPage;
constexpr int kStages = 2;
constexpr int kSoftmaxThreads = 128;
constexpr int kProducerWarp = 4, kMmaWarp = 5;
constexpr int kThreads = 192;
// Every operand is stored as 64-element (128-byte) column halves of [rows][128 B], 128-byte swizzled.
constexpr int kQHalfBytes = kBlockM * 128;       // Q: 128 rows x 64 dims, 16 KiB; two of them
constexpr int kQBytes = 2 * kQHalfBytes;
constexpr int kKvHalfBytes = kBlockN * 128;      // K (or V): kBlockN keys x 64 dims; two of them per operand
constexpr int kKvOperandBytes = 2 * kKvHalfBytes;
constexpr int kStageBytes = 2 * kKvOperandBytes; // K block + V block
constexpr int kTmemCols = 256;                   // per CTA; two CTAs share the SM's 512 columns
constexpr int kColS = 0, kColO = 2 * kBlockN;    // S buffers at columns 0 and kBlockN, O (128 columns) after them
constexpr int kAlignSlack = 256;                 // spare bytes in front of the operands (two CTAs must fit one SM)
static_assert(kBlockN % 64 == 0 && kColO + kD <= kTmemCols, "TMEM budget");
constexpr int kErrTimeout = 8;
constexpr float kRescaleThreshold = 8.f;     // log2 units
// One partial result: the accumulator as float4 [32 dim-quads][128 rows] (a warp stores 512 contiguous bytes), then
// the rows' running maxima and sums.
constexpr int kPartialFloats = kBlockM * kD + 2 * kBlockM;
// Merging one partial costs its reader about as much as kMergeCostBlocks blocks (64 KiB from L2 by one CTA);
// pieces shorter than sqrt(kMergeCostBlocks * longest tile) blocks would spend more on merging than they save.
constexpr float kMergeCostBlocks = 2.7f;
// What a tile costs besides its blocks -- loading its Q rows, draining the pipeline, normalising and storing (or parking)
// its rows -- in units of one block's time. The line that is cut into equal pieces counts every tile as its blocks plus
// this many units, so a CTA whose piece is made of many short tiles gets fewer blocks than one inside a long tile.
constexpr int kTileCost = 5;

// barrier indices
enum : int {
    // ONE tcgen05.commit per batch of MMAs, waited on by both of its consumers. With two commits in a row the second
    // arrival came about 900 clocks after the first -- not when its MMAs had finished but when the batch issued after
    // it had (measured with an idle lane polling the barrier) -- and the K tile two blocks ahead was requested that much
    // later, which stalled the MMA thread on every block.
    kBarKFull = 0,                    // [kStages] producer -> MMA: K block landed (transaction bytes)
    kBarVFull = kBarKFull + kStages,  // [kStages] producer -> MMA: V block landed
    kBarQKDone = kBarVFull + kStages, // [2] MMA (commit) -> softmax: S[buf] written; -> producer: K stage buf is free
    kBarPFull = kBarQKDone + 2,       // softmax (128) -> MMA: S read, P in tensor memory over it, O rescaled
                                      // ("S[buf] is free again" needs no barrier: it is the P arrival of two blocks
                                      // earlier, which the MMA thread has waited for)
    kBarPVDone = kBarPFull + 1,       // [2] MMA (commit) -> softmax: O stable; -> producer: V stage is free
    kBarQFull = kBarPVDone + 2,       // softmax (128) -> MMA: Q rows of the next fragment are in shared memory
    kBarMerge = kBarQFull + 1,        // bulk copy -> softmax: the other half of a split tile is in shared memory
    kNumBars = kBarMerge + 1
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
    int32_t n_seqs, nkvh, group, nh;
    const void *q;
    void *out;
    float scale_log2;
    int32_t *error_flag;
    float *partials;   // [2 * gridDim.x][kPartialFloats]
    int32_t *counters; // [gridDim.x], zero between launches
    int32_t out_wide;  // out is 32-byte aligned: rows are stored 32 bytes (a whole sector) per instruction
};

// ---- the line of blocks ------------------------------------------------------------------------------------------

struct SeqGeom {
    int q_start, q_len, kv_len, off, n_qb;
};

__device__ __forceinline__ SeqGeom seq_geom(const PrefillParams &p, int a) {
    SeqGeom g;
    if (p.contiguous) {
        g.q_start = 0;
        g.q_len = p.const_q_len;
        g.kv_len = max(p.const_kv_len, g.q_len);
    } else {
        g.q_start = p.q_starts[a];
        g.q_len = p.q_starts[a + 1] - g.q_start;
        g.kv_len = min(max(p.kv_lens[a], g.q_len), p.table_stride * kPage);
    }
    g.off = g.kv_len - g.q_len; // query t sees keys j <= t + off
    g.n_qb = (g.q_len + kBlockM - 1) / kBlockM;
    return g;
}

// keys any row of row block qb can see, and the 64-key blocks that hold them
__device__ __forceinline__ int tile_kv_hi(const SeqGeom &g, int qb) { return min(g.kv_len, qb * kBlockM + kBlockM + g.off); }
__device__ __forceinline__ int tile_blocks(const SeqGeom &g, int qb) { return (tile_kv_hi(g, qb) + kBlockN - 1) / kBlockN; }

// units of the line that a sequence takes: per tile its blocks, then kTileCost units that stand for no block
__device__ __forceinline__ int seq_blocks(const PrefillParams &p, const SeqGeom &g) {
    int per_head = 0;
    for (int qb = 0; qb < g.n_qb; ++qb) {
        per_head += tile_blocks(g, qb) + kTileCost;
    }
    return per_head * p.nh;
}

// Position on the line: every role of the CTA walks the same fragments with one of these.
struct Walker {
    int a;         // sequence
    int seq_begin; // index on the line of its first block
    int n_blocks;  // its blocks (all heads)
    SeqGeom g;
};

struct Fragment {
    int a, qb, h;
    int b0, b1;     // key blocks [b0, b1) of the tile
    int tile_nblk;  // blocks of the whole tile
    int tile_begin; // index on the line of the tile's block 0
};

// The fragment that starts at or after unit `pos` of the line and before piece_end: `pos` moves on to its first block
// (over the units at a tile's end that stand for no block). False when the piece holds no further block.
__device__ __forceinline__ bool locate(const PrefillParams &p, Walker &w, int &pos, int piece_end, Fragment &f) {
    while (pos < piece_end) {
        while (pos >= w.seq_begin + w.n_blocks && w.a + 1 < p.n_seqs) {
            w.seq_begin += w.n_blocks;
            ++w.a;
            w.g = seq_geom(p, w.a);
            w.n_blocks = seq_blocks(p, w.g);
        }
        int x = pos - w.seq_begin;
        int qb = 0, nb = tile_blocks(w.g, 0);
        while (x >= (nb + kTileCost) * p.nh && qb + 1 < w.g.n_qb) {
            x -= (nb + kTileCost) * p.nh;
            ++qb;
            nb = tile_blocks(w.g, qb);
        }
        const int h = min(x / (nb + kTileCost), p.nh - 1);
        const int b0 = x - h * (nb + kTileCost);
        if (b0 >= nb + kTileCost) {
            return false; // (past the end of the line: no caller asks)
        }
        if (b0 >= nb) { // behind the tile's last block: on to the next tile
            pos += nb + kTileCost - b0;
            continue;
        }
        f.a = w.a;
        f.qb = qb;
        f.h = h;
        f.b0 = b0;
        f.tile_nblk = nb;
        f.b1 = min(nb, b0 + (piece_end - pos));
        f.tile_begin = pos - b0;
        return true;
    }
    return false;
}

// Blackwell's wider scalar arithmetic for the softmax rows: a three-input maximum and two-wide f32 multiply-add / add
// (one instruction for two scores: these warps are short of issue slots, not of pipe throughput).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void fma2(float &x0, float &x1, float a0, float a1, float b, float c) { // x = a * b + c
    asm("{\n"
        ".reg .b64 ra, rb, rc, rd;\n"
        "mov.b64 ra, {%2, %3};\n"
        "mov.b64 rb, {%4, %4};\n"
        "mov.b64 rc, {%5, %5};\n"
        "fma.rn.f32x2 rd, ra, rb, rc;\n"
        "mov.b64 {%0, %1}, rd;\n"
        "}\n"
        : "=f"(x0), "=f"(x1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float &s0, float &s1, float a0, float a1) { // s += a
    asm("{\n"
        ".reg .b64 rs, ra;\n"
        "mov.b64 rs, {%0, %1};\n"
        "mov.b64 ra, {%2, %3};\n"
        "add.rn.f32x2 rs, rs, ra;\n"
        "mov.b64 {%0, %1}, rs;\n"
        "}\n"
        : "+f"(s0), "+f"(s1)
        : "f"(a0), "f"(a1));
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 2)
    paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_v,
                            PrefillParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t base_u32 = (raw_u32 + 1023u) & ~1023u; // swizzled operands need 1 KiB alignment
    unsigned char *base = smem_raw + (base_u32 - raw_u32);
    const uint32_t q_u32 = base_u32, kv_u32 = base_u32 + kQBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + kQBytes + kStages * kStageBytes);
    const uint32_t bars_u32 = smem_u32(bars);
    uint32_t *s_tmem_base = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem_base + 1);
    int *s_sched = reinterpret_cast<int *>(s_tmem_base + 2); // [16]: warp sums, totals, start of the piece, arrival order

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (base_u32 - raw_u32 > uint32_t(kAlignSlack)) { // cannot place the swizzled operands: report, do not run
        if (tid == 0) {
            atomicOr(p.error_flag, kErrTimeout);
        }
        return;
    }

    // ---- this CTA's piece of the line ----------------------------------------------------------------------------
    // (every CTA sums the sequences' blocks itself: a few loads per sequence, no launch in front of this one)
    int line_blocks = 0, longest_tile = 0;
    {
        int mine = 0, mine_max = 0;
        for (int a = tid; a < p.n_seqs; a += kThreads) {
            const SeqGeom g = seq_geom(p, a);
            mine += seq_blocks(p, g);
            mine_max = max(mine_max, g.n_qb > 0 ? tile_blocks(g, g.n_qb - 1) : 0);
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            mine += __shfl_xor_sync(0xffffffffu, mine, d);
            mine_max = max(mine_max, __shfl_xor_sync(0xffffffffu, mine_max, d));
        }
        if (lane == 0) {
            s_sched[warp] = mine;
            s_sched[6 + warp] = mine_max;
        }
        __syncthreads();
        for (int w = 0; w < kThreads / 32; ++w) {
            line_blocks += s_sched[w];
            longest_tile = max(longest_tile, s_sched[6 + w]);
        }
    }
    const int n_slots = int(gridDim.x);
    const int min_piece = int(ceilf(sqrtf(kMergeCostBlocks * float(longest_tile))));
    const int piece = max((line_blocks + n_slots - 1) / n_slots, max(min_piece, kTileCost + 1)); // units per CTA
    const int slot = int(blockIdx.x);
    const int piece_begin = slot * piece;
    if (piece_begin >= line_blocks) {
        return; // uniform over the CTA, before any mbarrier or TMEM allocation
    }
    const int piece_end = min(line_blocks, piece_begin + piece);
    {
        // the sequence that holds block piece_begin, by a block-wide scan over kThreads sequences at a time
        __syncthreads();
        int before = 0; // blocks of the sequences in front of this pass's
        for (int a0 = 0; a0 < p.n_seqs; a0 += kThreads) {
            const int a = a0 + tid;
            const int w_a = a < p.n_seqs ? seq_blocks(p, seq_geom(p, a)) : 0;
            int incl = w_a;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                incl += lane >= d ? up : 0;
            }
            if (lane == 31) {
                s_sched[warp] = incl;
            }
            __syncthreads();
            int warps_before = 0, round_total = 0;
            for (int w = 0; w < kThreads / 32; ++w) {
                warps_before += w < warp ? s_sched[w] : 0;
                round_total += s_sched[w];
            }
            const int excl = before + warps_before + incl - w_a;
            if (w_a > 0 && excl <= piece_begin && piece_begin < excl + w_a) {
                s_sched[12] = a;
                s_sched[13] = excl;
            }
            before += round_total;
            __syncthreads();
            if (before > piece_begin) {
                break;
            }
        }
    }
    Walker walker;
    walker.a = s_sched[12];
    walker.seq_begin = s_sched[13];
    walker.g = seq_geom(p, walker.a);
    walker.n_blocks = seq_blocks(p, walker.g);
    Fragment first_fragment;
    Walker first_walker = walker;
    {
        int pos0 = piece_begin;
        if (!locate(p, first_walker, pos0, piece_end, first_fragment)) {
            return; // the piece holds no block (the line's last units): uniform over the CTA, nothing set up yet
        }
    }

    auto load_q = [&](const Fragment &f, const SeqGeom &g, int first, int stride) {
        // Q rows of the tile, 16 bytes per store, into the K-major 128-byte-swizzled layout
        // [dims 0-63 | dims 64-127][128 rows][128 B]; rows past the chunk are zero. All loads first, then all stores:
        // the stores are volatile asm, which no load may pass, and one round trip per 16 bytes made a fragment
        // boundary cost six blocks' time.
        const char *q_base = static_cast<const char *>(p.q);
        constexpr int kMaxIter = kBlockM * 16 / kSoftmaxThreads; // the fewest threads that call this
        uint4 vals[kMaxIter];
#pragma unroll
        for (int it = 0; it < kMaxIter; ++it) {
            const int idx = first + it * stride;
            const int r = idx >> 4, cc = idx & 15;
            const int t = f.qb * kBlockM + r;
            vals[it] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < kBlockM * 16 && t < g.q_len) {
                vals[it] = *reinterpret_cast<const uint4 *>(q_base + ((long long)(g.q_start + t) * p.nh + f.h) * (kD * 2) + cc * 16);
            }
        }
#pragma unroll
        for (int it = 0; it < kMaxIter; ++it) {
            const int idx = first + it * stride;
            const int r = idx >> 4, cc = idx & 15;
            if (idx < kBlockM * 16) {
                const uint32_t dst = q_u32 + (cc >> 3) * kQHalfBytes + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "r"(vals[it].x), "r"(vals[it].y),
                             "r"(vals[it].z), "r"(vals[it].w)
                             : "memory");
            }
        }
    };

    // ---- set-up: barriers, TMEM, first Q tile, cleared K/V ring ----------------------------------------------
    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            const bool many = i == kBarPFull || i == kBarQFull; // (kBarMerge: one arrival, by the thread that starts the copies)
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
        // Everything above read only the launch's index arrays and set up on-chip state; q, the K/V rows of the chunk,
        // the workspace and the outputs belong to the stream's order: with launch overlap on, wait here for the kernel
        // directly before this one, and only then let the one behind this one start.
        grid_dependency_wait();
        grid_launch_dependents();
        load_q(first_fragment, first_walker.g, tid, kThreads);
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
        // ================================ producer: TMA tiles of K and V =========================================
        bool alive = true;
        int done = 0; // blocks of earlier fragments: ring stage and parity run on across fragments
        for (int pos = piece_begin; alive;) {
            Fragment f;
            if (!locate(p, walker, pos, piece_end, f)) {
                break;
            }
            const int n = f.b1 - f.b0;
            const int n_pages = (tile_kv_hi(walker.g, f.qb) + kPage - 1) / kPage;
            const int kvh = f.h / p.group;
            const int seq_row = (!p.contiguous && p.seq_ids) ? p.seq_ids[f.a] : f.a;
            const long long tbase = (long long)seq_row * p.table_stride;
            // Page numbers come 8 blocks (32 table entries, one 128-byte load) at a time, and the group after the
            // current one is requested a whole group early: a table load issued when its block is due costs more than
            // a block takes (measured: about 1300 clocks between a V tile and the next K tile, on the critical path
            // of every block).
            auto load_group = [&](int blk0) {
                const int idx = blk0 * kPagesPerBlock + lane;
                if (p.contiguous) {
                    return idx; // block b of the tensor is its tokens [64 b, 64 b + 64)
                }
                return idx < n_pages ? p.block_table[tbase + idx] : 0;
            };
            int group = load_group(f.b0), next_group = load_group(f.b0 + 8);
            for (int i = 0; i < n && alive; ++i) {
                const int gi = done + i, st = gi & 1;
                const int first = (f.b0 + i) * kPagesPerBlock;
                const int n_pg = min(kPagesPerBlock, n_pages - first);
                if (i > 0 && (i & 7) == 0) {
                    group = next_group;
                    next_group = load_group(f.b0 + i + 8);
                }
                int page = __shfl_sync(0xffffffffu, group, (i & 7) * kPagesPerBlock + (lane & (kPagesPerBlock - 1)));
                if (lane < n_pg && !p.contiguous && (page < 0 || page >= p.num_pages)) {
                    atomicOr(p.error_flag, kErrBadPage);
                    page = 0;
                }
                const int c3 = int((p.page0 + page) * 2); // K of the page; V is the next index
                const uint32_t dst = kv_u32 + st * kStageBytes + lane * 2048;
#pragma unroll
                for (int is_v = 0; is_v < 2; ++is_v) {
                    const int full = (is_v ? kBarVFull : kBarKFull) + st, empty = (is_v ? kBarPVDone : kBarQKDone) + st;
                    if (gi >= kStages && !wait_or_abort(bar(empty), uint32_t((gi >> 1) - 1) & 1u, s_abort)) {
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
                    if (lane < n_pg && is_v) {
                        // V: ONE box per page -- 64 dims x 16 tokens x the 2 halves of the row -- lands as
                        // [half][16 tokens][128 B], which is what the MN-major B operand of P.V reads 16 keys at a time
                        // (tokens past the end of a contiguous tensor read as 0)
                        const uint32_t at = kv_u32 + st * kStageBytes + kKvOperandBytes + lane * (2 * 2048);
                        if (p.contiguous) {
                            tma_load_4d(at, &tmap_v, 0, page * kPage, 0, kvh, bar(full));
                        } else {
                            tma_load_5d(at, &tmap_v, 0, 0, 0, kvh, c3 + 1, bar(full));
                        }
                    } else if (lane < n_pg) {
                        // K: the K-major B operand of Q.K^T wants the 64 keys of a block side by side in each 64-dim half,
                        // so a page is two boxes of 64 dims x 16 tokens
                        const uint32_t lo = dst, hi = lo + kKvHalfBytes; // dims 0-63, dims 64-127
                        if (p.contiguous) {
                            // [tokens][kv-heads][128] tensor: box = 64 dims x 1 head x 16 tokens; tokens past the end read as 0
                            tma_load_3d(lo, &tmap, 0, kvh, page * kPage, bar(full));
                            tma_load_3d(hi, &tmap, 64, kvh, page * kPage, bar(full));
                        } else {
                            tma_load_4d(lo, &tmap, 0, 0, kvh, c3, bar(full));
                            tma_load_4d(hi, &tmap, 64, 0, kvh, c3, bar(full));
                        }
                    }
                }
            }
            pos += n;
            done += n;
        }
    } else if (warp == kMmaWarp) {
        // ================================ MMA issuer (one thread) =============================================
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(kBf16, false, kBlockM, kBlockN);
            constexpr uint32_t idesc_pv = make_idesc(kBf16, true, kBlockM, kD);
            const uint32_t tmem_o = tmem_base + kColO;
            bool ok = true;
            auto issue_pv = [&](int gj, bool first_of_fragment) { // O (+)= P . V of the CTA's gj-th block
                if (!wait_or_abort(bar(kBarPFull), uint32_t(gj) & 1u, s_abort) ||
                    !wait_or_abort(bar(kBarVFull + (gj & 1)), uint32_t(gj >> 1) & 1u, s_abort)) {
                    return false;
                }
                tc_fence_after();
                const uint32_t v_u32 = kv_u32 + (gj & 1) * kStageBytes + kKvOperandBytes;
#pragma unroll
                for (int kk = 0; kk < kBlockN / 16; ++kk) {
                    // B = 16 keys (one page) x 128 dims of V, MN-major: 8-key groups 1 KiB apart, the page's two
                    // 64-dim halves 2 KiB apart, pages 4 KiB apart. A = P rows x 16 keys from tensor memory: 8 columns
                    // of packed pairs per step, in S buffer gj & 1
                    const uint64_t b = smem_desc_sw128(v_u32 + kk * (2 * 2048), 2048, 1024);
                    umma_f16_ts(tmem_o, tmem_base + kColS + (gj & 1) * kBlockN + kk * 8, b, idesc_pv,
                                (!first_of_fragment || kk > 0) ? 1u : 0u);
                }
                umma_commit(bar(kBarPVDone + (gj & 1)));
                return true;
            };
            int done = 0, frag_no = 0;
            for (int pos = piece_begin; ok; ++frag_no) {
                Fragment f;
                if (!locate(p, walker, pos, piece_end, f)) {
                    break;
                }
                const int n = f.b1 - f.b0;
                if (frag_no > 0) { // the softmax threads have stored this fragment's Q rows
                    ok = wait_or_abort(bar(kBarQFull), uint32_t(frag_no - 1) & 1u, s_abort);
                }
                for (int i = 0; i < n && ok; ++i) {
                    const int gi = done + i, st = gi & 1, buf = gi & 1;
                    ok = wait_or_abort(bar(kBarKFull + st), uint32_t(gi >> 1) & 1u, s_abort);
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
                    umma_commit(bar(kBarQKDone + buf));
                    if (i >= 1) {
                        ok = issue_pv(gi - 1, i == 1);
                    }
                }
                if (ok) {
                    ok = issue_pv(done + n - 1, n == 1);
                }
                pos += n;
                done += n;
            }
            if (!ok) {
                give_up();
            }
        }
    } else {
        // ================================ softmax: one query row per thread =====================================
        const int row = tid;                       // TMEM lane
        const uint32_t lane_base = uint32_t(warp * 32) << 16;
        const uint32_t tmem_o = tmem_base + lane_base + kColO;
        // A thread whose wait ran out stops computing but keeps walking the fragments, so that the named barrier and
        // the arrival counts below see all 128 threads every time.
        bool dead = false;
        int done = 0;
        for (int pos = piece_begin;;) {
            Fragment f;
            if (!locate(p, walker, pos, piece_end, f)) {
                break;
            }
            const SeqGeom g = walker.g;
            const int n = f.b1 - f.b0;
            const int t = f.qb * kBlockM + row;        // query index inside the chunk
            const int last_visible = t + g.off;        // keys j <= last_visible (and < kv_len) take part
            float m_used = -INFINITY, l = 0.f;
            for (int i = 0; i < n && !dead; ++i) {
                const int gi = done + i, buf = gi & 1;
                if (!wait_or_abort(bar(kBarQKDone + buf), uint32_t(gi >> 1) & 1u, s_abort)) {
                    dead = true;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_s = tmem_base + lane_base + kColS + buf * kBlockN;
                const int j0 = (f.b0 + i) * kBlockN;
                const int n_ok = min(min(last_visible, g.kv_len - 1) - j0 + 1, kBlockN); // visible columns are [0, n_ok)
                uint32_t sr[kBlockN / 32][32];
#pragma unroll
                for (int c = 0; c < kBlockN / 32; ++c) {
                    tmem_ld32_nowait(tmem_s + c * 32, sr[c]);
                }
                tmem_wait_ld();
                // Most blocks lie wholly below the diagonal: the whole warp then skips the mask (warp-uniform choice).
                // Otherwise the hidden scores become -inf and take the same path: 2^(-inf * scale - m) = 0. (A scale
                // that is not positive takes the slow path further down.)
                const bool plain = p.scale_log2 > 0.f;
                if (plain && !__all_sync(0xffffffffu, n_ok >= kBlockN)) {
#pragma unroll
                    for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                        for (int k = 0; k < 32; ++k) {
                            sr[c][k] = c * 32 + k < n_ok ? sr[c][k] : 0xff800000u;
                        }
                    }
                }
                // Row maximum as eight independent chains (a single chain of 64 dependent max operations would cost more
                // than the exponentials that follow).
                float mx8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    mx8[u] = -INFINITY;
                }
                if (plain) {
#pragma unroll
                    for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                        for (int k = 0; k < 16; ++k) {
                            mx8[k & 7] = max3(mx8[k & 7], __uint_as_float(sr[c][k]), __uint_as_float(sr[c][k + 16]));
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
                    alpha = fast_exp2(m_used - mx); // 0 on the fragment's first visible block
                    m_used = mx;
                }
                l *= alpha;
                // P = 2^(s - m) as 16-bit, computed into registers BEFORE waiting for the previous PV: only the stores
                // of P sit on the block-to-block dependency chain.
                const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
                uint32_t packed[kBlockN / 2];
                float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f; // independent sums: short dependency chains
                if (plain) {
#pragma unroll
                    for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                        for (int k = 0; k < 32; k += 2) {
                            float x0, x1;
                            fma2(x0, x1, __uint_as_float(sr[c][k]), __uint_as_float(sr[c][k + 1]), p.scale_log2, neg_m);
                            const float p0 = fast_exp2(x0);
                            const float p1 = fast_exp2(x1);
                            if (k & 2) {
                                add2(l2, l3, p0, p1);
                            } else {
                                add2(l0, l1, p0, p1);
                            }
                            packed[c * 16 + (k >> 1)] = pack2<kBf16>(p0, p1);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                        for (int k = 0; k < 32; k += 2) {
                            const float p0 =
                                (c * 32 + k < n_ok) ? fast_exp2(fmaf(__uint_as_float(sr[c][k]), p.scale_log2, neg_m)) : 0.f;
                            const float p1 = (c * 32 + k + 1 < n_ok)
                                                 ? fast_exp2(fmaf(__uint_as_float(sr[c][k + 1]), p.scale_log2, neg_m))
                                                 : 0.f;
                            l0 += p0;
                            l1 += p1;
                            packed[c * 16 + (k >> 1)] = pack2<kBf16>(p0, p1);
                        }
                    }
                }
                l += (l0 + l1) + (l2 + l3);
                // PV of the previous block (of this fragment or the one before) must be finished before O is rescaled.
                // The hand-over of P would not need this wait, but every phase of the barrier has to be observed in
                // order: a parity wait cannot tell "two phases behind" from "done", and a thread that skipped phases
                // passed the final wait before the last two products had finished (rare wrong rows in tiles that ran
                // alone on their SM).
                const bool any_grow = __any_sync(0xffffffffu, grow);
                if (gi >= 1) {
                    if (!wait_or_abort(bar(kBarPVDone + ((gi - 1) & 1)), uint32_t((gi - 1) >> 1) & 1u, s_abort)) {
                        dead = true;
                        break;
                    }
                    tc_fence_after();
                    if (i >= 1 && any_grow) { // (the first PV of a fragment overwrites O: nothing to rescale before it)
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
                // 64 keys = 32 columns of packed pairs over the first half of S[buf]; the same arrival tells the tensor
                // pipe that P is there and (S having been read above) that the buffer may be rewritten after this PV
                tmem_st32_words(tmem_s, packed);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar(kBarPFull));
            }
            // ---- Q rows of the next fragment: every QK^T of this one has finished (its last S was read above) -------
            bool more; // another fragment follows in this CTA (uniform over the CTA)
            {
                Walker wn = walker;
                Fragment fn;
                int pos_n = pos + n;
                more = locate(p, wn, pos_n, piece_end, fn);
                if (more && !dead) {
                    load_q(fn, wn.g, tid, kSoftmaxThreads);
                    fence_proxy_async_smem();
                    mbar_arrive(bar(kBarQFull));
                }
            }
            // ---- epilogue of the fragment ---------------------------------------------------------------------------
            if (!dead && !wait_or_abort(bar(kBarPVDone + ((done + n - 1) & 1)), uint32_t((done + n - 1) >> 1) & 1u, s_abort)) {
                dead = true;
            }
            tc_fence_after();
            const bool whole = f.b0 == 0 && f.b1 == f.tile_nblk;
            char *out_row = static_cast<char *>(p.out) + ((long long)(g.q_start + t) * p.nh + f.h) * (kD * 2);
            bool store_rows = whole, staged = false;
            float w_own = 1.f, l_all = l, m_all = m_used;
            float w_oth[4] = {0.f, 0.f, 0.f, 0.f}; // staged merge: weights of the other fragments, in the order of their CTAs
            const int first_slot = f.tile_begin / piece, last_slot = (f.tile_begin + f.tile_nblk - 1) / piece;
            const int n_others = last_slot - first_slot, own_at = slot - first_slot; // fragments besides this one; those before it
            int chunks_per_trip = 4; // staged merge: 32-column chunks of every other fragment fetched per trip (4 / n_others)
            if (!whole) {
                // unnormalised accumulator + (max, sum) of the rows into this CTA's workspace slot: slot 1 for the
                // fragment that begins its tile (and continues in the next CTA), slot 0 for one that began earlier
                float *part = p.partials + (long long)(slot * 2 + (f.b0 == 0 ? 1 : 0)) * kPartialFloats;
                if (!dead) {
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {
                        float v[32];
                        tmem_ld32(tmem_o + c4 * 32, v);
#pragma unroll
                        for (int q8 = 0; q8 < 8; ++q8) {
                            reinterpret_cast<float4 *>(part)[(c4 * 8 + q8) * kBlockM + row] =
                                make_float4(v[q8 * 4], v[q8 * 4 + 1], v[q8 * 4 + 2], v[q8 * 4 + 3]);
                        }
                    }
                    part[kBlockM * kD + row] = m_used;
                    part[kBlockM * kD + kBlockM + row] = l;
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (tid == 0) {
                    const int n_frags = last_slot - first_slot + 1;
                    const int before = atomicAdd(p.counters + first_slot, 1);
                    const bool last = before == n_frags - 1;
                    if (last) {
                        p.counters[first_slot] = 0; // ready for the next launch
                    }
                    s_sched[14] = last ? 1 : 0;
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                store_rows = s_sched[14] != 0;
                // The usual merge: the CTA's last fragment begins a tile that the next CTA finished long ago (or, for a
                // tile longer than a piece, that the next CTAs are spread over). The operands and Q are no longer
                // needed, so the other fragments (64 KiB each + maxima and sums) are fetched into their place by bulk
                // copies and combined from shared memory: one trip to L2 for one other fragment, two for two, four
                // for three or four (the K/V ring holds 64 KiB) instead of six dependent ones. Same arithmetic, in the
                // same order, as the general path below.
                staged = store_rows && !more && n_others <= 4;
                if (staged) {
                    chunks_per_trip = 4 / n_others; // 4, 2, 1, 1
                    if (tid == 0) {
                        __threadfence();
                        asm volatile("fence.proxy.async;\n" ::: "memory"); // generic-proxy writes of another SM -> bulk read
                        mbar_arrive_expect_tx(bar(kBarMerge), uint32_t(n_others) * uint32_t(chunks_per_trip * 16384 + 2 * kBlockM * 4));
                        int j = 0;
                        for (int s2 = first_slot; s2 <= last_slot; ++s2) {
                            if (s2 == slot) {
                                continue;
                            }
                            const float *other =
                                p.partials + (long long)(s2 * 2 + (s2 * piece <= f.tile_begin ? 1 : 0)) * kPartialFloats;
                            for (int u = 0; u < chunks_per_trip; ++u) {
                                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                                                 kv_u32 + (j * chunks_per_trip + u) * 16384),
                                             "l"(other + u * 4096), "r"(16384), "r"(bar(kBarMerge))
                                             : "memory");
                            }
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                                             q_u32 + j * (2 * kBlockM * 4)),
                                         "l"(other + kBlockM * kD), "r"(2 * kBlockM * 4), "r"(bar(kBarMerge))
                                         : "memory");
                            ++j;
                        }
                    }
                    if (!dead && !wait_or_abort(bar(kBarMerge), 0u, s_abort)) {
                        dead = true;
                    }
                    float m_oth[4], l_oth[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        m_oth[j] = -INFINITY;
                        l_oth[j] = 0.f;
                        if (j < n_others) {
                            asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(m_oth[j]) : "r"(q_u32 + j * (2 * kBlockM * 4) + row * 4) : "memory");
                            asm volatile("ld.shared.f32 %0, [%1];\n"
                                         : "=f"(l_oth[j])
                                         : "r"(q_u32 + j * (2 * kBlockM * 4) + (kBlockM + row) * 4)
                                         : "memory");
                        }
                        m_all = fmaxf(m_all, m_oth[j]);
                    }
                    w_own = m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_all);
                    l_all = 0.f;
#pragma unroll
                    for (int j = 0; j <= 4; ++j) { // the others in the order of their CTAs, this fragment in its place
                        if (j == own_at) {
                            l_all = fmaf(l, w_own, l_all);
                        }
                        if (j < 4 && j < n_others) {
                            w_oth[j] = m_oth[j] == -INFINITY ? 0.f : fast_exp2(m_oth[j] - m_all);
                            l_all = fmaf(l_oth[j], w_oth[j], l_all);
                        }
                    }
                } else if (store_rows && !dead) {
                    __threadfence();
                    // merge the other fragments' rows into this one's: weights 2^(m_i - m) in the log2 domain
                    for (int s2 = first_slot; s2 <= last_slot; ++s2) {
                        if (s2 != slot) {
                            const float *other =
                                p.partials + (long long)(s2 * 2 + (s2 * piece <= f.tile_begin ? 1 : 0)) * kPartialFloats;
                            m_all = fmaxf(m_all, __ldcg(other + kBlockM * kD + row));
                        }
                    }
                    // (sums run over the fragments in the order of their CTAs, this one's terms in its place: the
                    // result does not depend on which fragment happened to arrive last)
                    w_own = m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_all);
                    l_all = 0.f;
                    for (int s2 = first_slot; s2 <= last_slot; ++s2) {
                        if (s2 != slot) {
                            const float *other =
                                p.partials + (long long)(s2 * 2 + (s2 * piece <= f.tile_begin ? 1 : 0)) * kPartialFloats;
                            const float m2 = __ldcg(other + kBlockM * kD + row);
                            const float w2 = m2 == -INFINITY ? 0.f : fast_exp2(m2 - m_all);
                            l_all = fmaf(__ldcg(other + kBlockM * kD + kBlockM + row), w2, l_all);
                        } else {
                            l_all = fmaf(l, w_own, l_all);
                        }
                    }
                }
            }
            if (store_rows && (staged || !dead)) {
                const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    if (staged && c4 > 0 && c4 % chunks_per_trip == 0) {
                        // next trip: everybody has read the chunks in shared memory (all 128 threads meet here, also
                        // those that have given up), then one thread asks for the next ones
                        asm volatile("bar.sync 1, 128;\n" ::: "memory");
                        if (tid == 0) {
                            asm volatile("fence.proxy.async;\n" ::: "memory"); // reads above -> the copies' writes
                            mbar_arrive_expect_tx(bar(kBarMerge), uint32_t(n_others) * uint32_t(chunks_per_trip * 16384));
                            int j = 0;
                            for (int s2 = first_slot; s2 <= last_slot; ++s2) {
                                if (s2 == slot) {
                                    continue;
                                }
                                const float *other =
                                    p.partials + (long long)(s2 * 2 + (s2 * piece <= f.tile_begin ? 1 : 0)) * kPartialFloats;
                                for (int u = 0; u < chunks_per_trip; ++u) {
                                    asm volatile(
                                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                                            kv_u32 + (j * chunks_per_trip + u) * 16384),
                                        "l"(other + (c4 + u) * 4096), "r"(16384), "r"(bar(kBarMerge))
                                        : "memory");
                                }
                                ++j;
                            }
                        }
                        if (!dead && !wait_or_abort(bar(kBarMerge), uint32_t(c4 / chunks_per_trip) & 1u, s_abort)) {
                            dead = true;
                        }
                    }
                    if (dead) {
                        continue;
                    }
                    float v[32];
                    tmem_ld32(tmem_o + c4 * 32, v);
                    if (staged) {
                        const uint32_t chunk_u32 = kv_u32 + uint32_t(c4 % chunks_per_trip) * 16384u + uint32_t(row) * 16u;
#pragma unroll
                        for (int q8 = 0; q8 < 8; ++q8) {
                            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                            for (int j = 0; j <= 4; ++j) {
                                if (j == own_at) {
                                    acc.x = fmaf(v[q8 * 4], w_own, acc.x);
                                    acc.y = fmaf(v[q8 * 4 + 1], w_own, acc.y);
                                    acc.z = fmaf(v[q8 * 4 + 2], w_own, acc.z);
                                    acc.w = fmaf(v[q8 * 4 + 3], w_own, acc.w);
                                }
                                if (j < 4 && j < n_others) {
                                    float4 o;
                                    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                                                 : "=f"(o.x), "=f"(o.y), "=f"(o.z), "=f"(o.w)
                                                 : "r"(chunk_u32 + uint32_t(j * chunks_per_trip) * 16384u + uint32_t(q8 * kBlockM) * 16u)
                                                 : "memory");
                                    acc.x = fmaf(o.x, w_oth[j], acc.x);
                                    acc.y = fmaf(o.y, w_oth[j], acc.y);
                                    acc.z = fmaf(o.z, w_oth[j], acc.z);
                                    acc.w = fmaf(o.w, w_oth[j], acc.w);
                                }
                            }
                            v[q8 * 4] = acc.x;
                            v[q8 * 4 + 1] = acc.y;
                            v[q8 * 4 + 2] = acc.z;
                            v[q8 * 4 + 3] = acc.w;
                        }
                    } else if (!whole) {
                        float own[32];
#pragma unroll
                        for (int k = 0; k < 32; ++k) {
                            own[k] = v[k];
                            v[k] = 0.f;
                        }
                        for (int s2 = first_slot; s2 <= last_slot; ++s2) {
                            if (s2 == slot) {
#pragma unroll
                                for (int k = 0; k < 32; ++k) {
                                    v[k] = fmaf(own[k], w_own, v[k]);
                                }
                            } else {
                                const float *other =
                                    p.partials + (long long)(s2 * 2 + (s2 * piece <= f.tile_begin ? 1 : 0)) * kPartialFloats;
                                const float m2 = __ldcg(other + kBlockM * kD + row);
                                const float w2 = m2 == -INFINITY ? 0.f : fast_exp2(m2 - m_all);
#pragma unroll
                                for (int q8 = 0; q8 < 8; ++q8) {
                                    const float4 o =
                                        __ldcg(reinterpret_cast<const float4 *>(other) + (c4 * 8 + q8) * kBlockM + row);
                                    v[q8 * 4] = fmaf(o.x, w2, v[q8 * 4]);
                                    v[q8 * 4 + 1] = fmaf(o.y, w2, v[q8 * 4 + 1]);
                                    v[q8 * 4 + 2] = fmaf(o.z, w2, v[q8 * 4 + 2]);
                                    v[q8 * 4 + 3] = fmaf(o.w, w2, v[q8 * 4 + 3]);
                                }
                            }
                        }
                    }
                    if (t < g.q_len && p.out_wide) {
                        // a thread owns a row: a 16-byte store fills half a 32-byte sector and the other half comes
                        // with the next instruction; 32-byte stores halve the write transactions of the epilogue
#pragma unroll
                        for (int q2 = 0; q2 < 2; ++q2) {
                            uint32_t w[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                w[e] = pack2<kBf16>(v[q2 * 16 + 2 * e] * inv, v[q2 * 16 + 2 * e + 1] * inv);
                            }
                            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"l"(out_row + c4 * 64 + q2 * 32),
                                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                                         : "memory");
                        }
                    } else if (t < g.q_len) {
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
            tc_fence_before(); // the O reads above come before the next fragment's P arrival in program order
            pos += n;
            done += n;
        }
        if (dead && lane == 0) {
            give_up();
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

// operands + barriers + TMEM-address / abort words + scheduling words; kAlignSlack bytes for the 1 KiB alignment of the
// operand area (the dynamic window itself starts aligned when the kernel has no static shared memory)
constexpr size_t kSmemBytes = kAlignSlack + kQBytes + kStages * kStageBytes + kNumBars * sizeof(uint64_t) + 8 + 16 * sizeof(int);

// CTAs of the fixed grid: two per SM
int prefill_slots() {
    static int slots[64] = {};
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    int &n = slots[dev & 63];
    if (n == 0) {
        int sms = 0;
        LLAISYS_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        n = 2 * (sms > 0 ? sms : 1);
    }
    return n;
}

template <bool kBf16>
void launch(cudaStream_t s, const CUtensorMap &tmap, const CUtensorMap &tmap_v, const PrefillParams &p, int grid, bool overlap) {
    static std::once_flag once[64];
    int dev = 0;
    LLAISYS_CUDA_CHECK(cudaGetDevice(&dev));
    std::call_once(once[dev & 63], [] {
        LLAISYS_CUDA_CHECK(cudaFuncSetAttribute(paged_prefill_tc_kernel<kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                int(kSmemBytes)));
    });
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(unsigned(kThreads));
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = overlap ? 1 : 0;
    LLAISYS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, paged_prefill_tc_kernel<kBf16>, tmap, tmap_v, p));
}

} // namespace

void attention_prefill_tc_scratch(size_t *floats, size_t *counters) {
    const size_t slots = size_t(prefill_slots());
    *floats = 2 * slots * size_t(kPartialFloats);
    *counters = slots;
}

int make_kv_tile_tensor_map(void *out_256_bytes, void *pool_base, uint64_t total_rows, uint32_t nkvh,
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
    // The second map is for V: a 5-D view [page-and-K|V][kv-head][half of the row][slot][64 elements] whose box is a whole
    // tile as two 64-dim halves, 64 x 16 x 2 (4 KiB): one copy per page instead of two.
    const cuuint64_t dims5[5] = {64, cuuint64_t(kPage), 2, cuuint64_t(nkvh), cuuint64_t(total_rows / (kPage * nkvh))};
    const cuuint64_t strides5[4] = {cuuint64_t(kD * 2), 128, cuuint64_t(kPage * kD * 2), cuuint64_t(kPage * kD * 2) * nkvh};
    const cuuint32_t box5[5] = {64, cuuint32_t(kPage), 2, 1, 1};
    const cuuint32_t elem_strides5[5] = {1, 1, 1, 1, 1};
    CUtensorMap map_v;
    const CUresult rc_v =
        encode(&map_v, dtype == LLAISYS_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
               pool_base, dims5, strides5, box5, elem_strides5, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc_v != CUDA_SUCCESS) {
        return -1;
    }
    static_assert(sizeof(CUtensorMap) == 128, "two maps in 256 bytes");
    memcpy(out_256_bytes, &map, sizeof(map));
    memcpy(static_cast<unsigned char *>(out_256_bytes) + sizeof(map), &map_v, sizeof(map_v));
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

// The same tensor for V: 4-D (64 dims, tokens, half of the row, kv-head) with a box of 64 x 16 x 2 x 1, one copy per 16 tokens.
bool contiguous_v_map(CUtensorMap *out, const void *base, const KVView &kv, uint64_t tokens, bool bf16) {
    EncodeTiledFn encode = prefill_encode_fn();
    if (encode == nullptr || tokens == 0 || tokens >= (uint64_t(1) << 31)) {
        return false;
    }
    const cuuint64_t dims[4] = {64, cuuint64_t(tokens), 2, cuuint64_t(kv.nkvh)};
    const cuuint64_t strides[3] = {cuuint64_t(kv.token_stride) * 2, 128, cuuint64_t(kv.head_stride) * 2};
    const cuuint32_t box[4] = {64, cuuint32_t(kPage), 2, 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    return encode(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base),
                  dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace

int attention_prefill_tc(stream_t stream, llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch,
                         const void *q, float scale, const AttnOut &out, const AttnScratch &scratch) {
    int32_t *error_flag = scratch.error_flag;
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
    p.q = q;
    p.out = out.out;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_flag = error_flag;
    // the workspace of the split tiles: two partial results per CTA and one arrival counter
    const int grid = prefill_slots();
    if (scratch.partials == nullptr || scratch.counters == nullptr ||
        scratch.partials_floats < 2 * size_t(grid) * size_t(kPartialFloats) || scratch.counters_len < size_t(grid) ||
        reinterpret_cast<uintptr_t>(scratch.partials) % 16 != 0) {
        return -1;
    }
    p.out_wide = reinterpret_cast<uintptr_t>(out.out) % 32 == 0 ? 1 : 0;
    p.partials = scratch.partials;
    p.counters = scratch.counters;
    CUtensorMap tmap, tmap_v;
    if (paged) {
        memcpy(&tmap, kv.tma_tile_desc, sizeof(tmap));
        memcpy(&tmap_v, static_cast<const unsigned char *>(kv.tma_tile_desc) + sizeof(tmap), sizeof(tmap_v));
    } else if (!contiguous_kv_map(&tmap, kv.k_base, kv, uint64_t(batch.const_kv_len), bf16) ||
               !contiguous_v_map(&tmap_v, kv.v_base, kv, uint64_t(batch.const_kv_len), bf16)) {
        return -1;
    }
    auto s = static_cast<cudaStream_t>(stream);
    if (bf16) {
        launch<true>(s, tmap, tmap_v, p, grid, kv.overlap_launch);
    } else {
        launch<false>(s, tmap, tmap_v, p, grid, kv.overlap_launch);
    }
    check_launch("paged_prefill_tc");
    return 0;
}

} // namespace llaisys::kernels
