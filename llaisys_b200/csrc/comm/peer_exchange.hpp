// Exchange of split-KV attention partials between the GPUs of one node through peer memory instead of a collective
// library: every rank owns a buffer of per-rank slots that all the others map (CUDA IPC) and write straight into over
// NVLink; a flag per writer, stamped with the step number, tells the owner when a slot is complete.
//
// One step on rank r (all on the caller's stream, capturable in a CUDA graph):
//   push    one CTA per destination: copy the local partial (o, m, l rows) into slot r of that rank's buffer (plain
//           peer stores), system-scope fence, then flag[r] = step there;
//   merge   wait (bounded) until all of this rank's flags carry the step, log-sum-exp merge the slots; the last CTA to
//           finish moves the device-side step counter on.
// Slots are double-buffered by the step's parity: a rank can run at most one step ahead of the slowest (its next wait
// needs that rank's next push), so a writer never overwrites a slot that is still being merged. No kernel waits
// without a limit: a wait that runs out sets the error word and the merge runs on what is there.
// New code: the reference has no multi-GPU path (README.md:426-427 names it as future work).
#pragma once

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
    // Device buffer the local partial decode writes to ([rows][d + 2] floats, at most slotFloats()).
    float *localPartial() const { return _local_part; }
    // push + merge for n_rows rows of head dimension d; out is [n_rows, d] of dtype.
    void exchangeAndMerge(llaisysStream_t stream, llaisysDataType_t dtype, void *out, int n_rows, int d);
    // Synchronises the stream, returns and clears the error word (0 = fine, 1 = a wait for a peer ran out).
    int status(llaisysStream_t stream);

private:
    int _rank, _world;
    size_t _slot_floats;
    bool _connected = false;
    unsigned char *_base = nullptr;      // this rank's allocation
    float *_local_part = nullptr;        // separate allocation: the decode kernel's output
    std::vector<unsigned char *> _peer;  // mapped bases, [_rank] = _base
    size_t _flags_offset = 0, _epoch_offset = 0, _error_offset = 0, _bytes = 0;
};

} // namespace llaisys::comm
