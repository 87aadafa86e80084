// Plain-data argument blocks shared by the CPU loops and the CUDA kernels of the attention path.
// Everything here is host-compilable (no CUDA types) so the operator layer can stay ordinary C++.
#pragma once

#include "llaisys.h"

#include <cstddef>
#include <cstdint>

namespace llaisys::kernels {

// Where the K and V rows of a sequence live. One description covers both layouts on the path:
//   paged pool   pool[page][K|V][kvh][slot][d]  -> page_stride = 2*nkvh*ps*d, head_stride = ps*d, token_stride = d,
//                v_base = k_base + nkvh*ps*d, block_table maps (sequence row, block) -> physical page;
//   contiguous   k[total, nkvh, d] as the legacy operator receives it
//                -> page_stride = ps*nkvh*d, head_stride = d, token_stride = nkvh*d, block_table = nullptr
//                (block b IS page b).
struct KVView {
    void *k_base = nullptr; // element (page 0, kv-head 0, slot 0, dim 0) of K (written only by append)
    void *v_base = nullptr; // same for V
    int64_t page_stride = 0;      // all strides in elements
    int64_t head_stride = 0;
    int64_t token_stride = 0;
    const int32_t *block_table = nullptr; // [rows][table_stride] on the executing device, or nullptr
    int32_t table_stride = 0;
    int32_t page_size = 16;
    int32_t num_pages = 0; // physical pages addressable through this view (bounds check)
    int32_t nkvh = 0;
    int32_t d = 0;
    // Optional TMA view of the same memory (page pools only): a 128-byte tensor-map blob in HOST memory over the
    // whole multi-layer pool, and the index of this layer's page 0 in it (layer * num_pages).
    // Launch append / decode with programmatic stream serialisation: the kernel's set-up and its first K/V copies may
    // overlap the tail of the previous kernel on the stream. Contract for the caller: index arrays and block tables were
    // written before that previous kernel started (K/V rows, q and outputs are only touched after it completed).
    bool overlap_launch = false;
    const void *tma_desc = nullptr;      // box = K and V of a page, 64 dims (decode)
    const void *tma_tile_desc = nullptr; // prefill, two maps of 128 bytes: box = one half-tile, 16 slots x 64 dims (K); box = a
                                         // tile as its two halves, 16 slots x 64 dims x 2 (V)
    int64_t tma_page0 = 0;
};

// Which queries attend to which sequences. Arrays live on the executing device; a null array selects the
// scalar that follows it (the legacy single-sequence operator has no arrays to pass).
struct AttnBatch {
    const int32_t *seq_ids = nullptr;  // [n_seqs] row of block_table per sequence; null: row i for sequence i
    const int32_t *kv_lens = nullptr;  // [n_seqs]; null: every sequence has const_kv_len tokens
    const int32_t *q_starts = nullptr; // [n_seqs + 1] first query row of each sequence; null: const_q_len each
    // The same seq_ids / kv_lens in HOST memory, for a caller that has them there anyway: the TMA decode kernel then takes
    // them by value with the launch (batches of at most 256 sequences) and the device arrays above may be null.
    const int32_t *host_seq_ids = nullptr;
    const int32_t *host_kv_lens = nullptr;
    int32_t const_kv_len = 0;
    int32_t const_q_len = 1;
    int32_t n_seqs = 0;
    int32_t total_q = 0; // rows of q / out
    int32_t max_q_len = 1;
    int32_t max_kv_len = 0;
    int32_t nh = 0;
};

// Output selection: `out` [total_q, nh, d] in the KV dtype, or `part` float [total_q, nh, d + 2] holding the
// locally normalised output followed by m (max scaled score, natural-log units) and l (sum of exp(score - m)).
struct AttnOut {
    void *out = nullptr;
    float *part = nullptr;
    const struct PeerSink *peers = nullptr; // decode over a page pool only: partial rows go to exchange slots instead
};

// Exchange buffers of a KV-range split across the GPUs of a node, as rank `rank` sees them: table[r] (an array in
// device memory) is rank r's buffer, peer memory for r != rank, and `own` is table[rank]. A buffer holds 2 (step
// parity) x world slots of slot_floats 8-byte words -- slot s of parity p is written by rank s; a word is a float and,
// beside it, the number of the step it belongs to, so that a reader can tell a current value from a stale one without
// any flag or fence -- then, at epoch_offset bytes, the step counter (merges completed). `rows` is local memory for
// this rank's rows [n_rows][d + 2] on their way out: the kernel completes a row there and copies it to every rank.
struct PeerSink {
    unsigned char *const *table = nullptr;
    unsigned char *own = nullptr;
    float *rows = nullptr;
    int32_t world = 0, rank = 0;
    size_t slot_floats = 0, epoch_offset = 0;
};

// Device-side scratch a launch may use (split-KV partials and arrival counters); owned by the caller.
struct AttnScratch {
    float *partials = nullptr;    // float [capacity]
    size_t partials_floats = 0;
    int32_t *counters = nullptr;  // int32 [counters_len], all zero between launches
    size_t counters_len = 0;
    int32_t *error_flag = nullptr; // set non-zero when a kernel skipped an out-of-range page / position
};

using stream_t = void *;

} // namespace llaisys::kernels
