// Exchange of split-KV attention partials between the GPUs of one node through peer memory instead of a collective
// library: every rank owns a buffer of per-rank slots that all the others map (CUDA IPC) and write straight into over
// NVLink. A slot is made of 8-byte words, each a float and, beside it, the number of the step it belongs to: written and
// read as one aligned access, the word is its own flag, so nothing in the exchange needs a fence, a separate flag or a
// count of finished rows (system-scope fences cost this GPU about 20 us apiece).
//
// One step on rank r (all on the caller's stream, capturable in a CUDA graph):
//   push    done by the TMA decode kernel itself (attention_decode_tma.cu, PeerSink): the CTA that completes a pair's
//           rows -- alone, or as the last of the CTAs that share the pair -- stores their words into slot r of EVERY
//           rank's buffer (plain peer stores, one warp, while the CTA's other warps stream on). Pools the TMA kernel
//           does not serve write the partial locally and a push kernel (one CTA per destination) forwards it;
//   merge   starts under the decode kernel (programmatic launch), asks for a row's words of all ranks at once and again
//           until each carries the step (bounded), log-sum-exp merges the slots; the last CTA to finish moves the
//           device-side step counter on.
// Slots are double-buffered by the step's parity: a rank can run at most one step ahead of the slowest (its next merge
// needs that rank's next values), so a writer never overwrites a slot that is still being merged, and a word left from
// two steps ago carries the wrong step. No kernel waits without a limit: a wait that runs out sets the error word and
// the merge runs on what is there -- the output of such a step is undefined, and because the ranks' step counters have
// then diverged the exchange must be destroyed and created again (by every rank) before the next step.
// New code: the reference has no multi-GPU path (README.md:426-427 names it as future work).
#pragma once

#include "../kernels/args.hpp"
#include "llaisys.h"

#include <cstddef>
#include <cstdint>
#include <vector>

namespace llaisys::comm {

constexpr int kMaxPeers = 16;
constexpr size_t kIpcHandleBytes = 64;

class PeerExchange {
public:
    // slot_floats: capacity of one rank's partial, in floats (rows * (head_dim + 2)). The calling thread's current CUDA
    // device must be the rank's device.
    PeerExchange(int rank, int world, size_t slot_floats);
    ~PeerExchange();
    PeerExchange(const PeerExchange &) = delete;
    PeerExchange &operator=(const PeerExchange &) = delete;

    int rank() const { return _rank; }
    int world() const { return _world; }
    size_t slotFloats() const { return _slot_floats; }
    void localHandle(void *out_64_bytes) const;
    // handles: world * 64 bytes, entry i from rank i (the own entry is ignored). Collective: call on every rank.
    void connect(const void *handles);
    // Unmaps the other ranks' buffers (after synchronising the device). A rank's buffer should only be released once
    // every other rank has unmapped it: disconnect on every rank, meet, then destroy.
    void disconnect();
    // Device buffer the local partial decode writes to ([rows][d + 2] floats, at most slotFloats()).
    float *localPartial() const { return _local_part; }
    // The buffers as the decode kernel needs them to store its partial rows at every rank itself.
    kernels::PeerSink sink() const;
    // Forwards n_rows rows of localPartial() to every rank (for kernels that cannot store there themselves).
    void push(llaisysStream_t stream, int n_rows, int d);
    // Takes every rank's values of this step as they arrive (bounded waits), merges them into out [n_rows, d] of dtype,
    // moves the step on.
    void merge(llaisysStream_t stream, llaisysDataType_t dtype, void *out, int n_rows, int d);
    // Polls (about half a microsecond each) after which a wait for a peer gives up; the default is about a second.
    void setWaitLimit(uint32_t polls);
    // Synchronises the stream, returns and clears the error word (0 = fine, 1 = a wait for a peer ran out).
    int status(llaisysStream_t stream);

private:
    int _rank, _world;
    size_t _slot_floats;
    bool _connected = false;
    unsigned char *_base = nullptr;      // this rank's allocation
    float *_local_part = nullptr;        // separate allocation: the decode kernel's output
    std::vector<unsigned char *> _peer;  // mapped bases, [_rank] = _base
    size_t _epoch_offset = 0, _error_offset = 0, _table_offset = 0, _bytes = 0;
    void writeTable();
    uint32_t _spin_limit = 2u << 20;
};

} // namespace llaisys::comm
