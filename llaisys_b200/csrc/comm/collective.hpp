// The one collective tensor parallelism needs: an in-place sum all-reduce of an activation buffer across the ranks
// that share a model. Two implementations behind one interface: NCCL on the rank's CUDA stream (the library is opened
// with dlopen at first use, so a process that already carries one -- PyTorch ships its own -- shares it), and a host
// callback for CPU runs and tests (the caller's function does the exchange, e.g. through a gloo process group).
// New code: the reference names NCCL / MPI tensor parallelism as future work (README.md:426-427).
#pragma once

#include "llaisys.h"

#include <cstddef>
#include <memory>

namespace llaisys::comm {

// In-place sum of `count` elements of `dtype` (llaisysDataType_t value) at `buf` (host memory) over all ranks;
// returns 0 on success.
using AllReduceCallback = int (*)(void *buf, size_t count, int dtype, void *user);

constexpr size_t kUniqueIdBytes = 128;

class Collective {
public:
    virtual ~Collective() = default;
    virtual void allReduceSum(void *buf, size_t count, llaisysDataType_t dtype, llaisysStream_t stream) = 0;
    int rank() const { return _rank; }
    int world() const { return _world; }

    // The calling thread's current CUDA device must be the rank's device.
    static std::unique_ptr<Collective> nccl(const void *unique_id, int rank, int world);
    static std::unique_ptr<Collective> callback(AllReduceCallback fn, void *user, int rank, int world);

protected:
    Collective(int rank, int world) : _rank(rank), _world(world) {}
    int _rank, _world;
};

// Fills 128 bytes with a fresh NCCL unique id (rank 0 makes one and sends it to the others by any host channel).
void ncclUniqueIdBytes(void *out);

} // namespace llaisys::comm
