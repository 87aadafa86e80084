// NCCL implementation of the all-reduce behind comm::Collective (see collective.hpp).
#include "collective.hpp"

#include "../kv/paged_kv.hpp"
#include "llaisys/paged_kv.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <string>

namespace llaisys::comm {

namespace {

[[noreturn]] void fail(int code, const std::string &msg) { throw kv::StatusError(code, msg); }

struct NcclApi {
    decltype(&ncclGetUniqueId) get_unique_id = nullptr;
    decltype(&ncclCommInitRank) comm_init_rank = nullptr;
    decltype(&ncclAllReduce) all_reduce = nullptr;
    decltype(&ncclCommDestroy) comm_destroy = nullptr;
    decltype(&ncclGetErrorString) error_string = nullptr;
    bool ok = false;
};

const NcclApi &nccl_api() {
    static const NcclApi api = [] {
        NcclApi a;
        void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (lib == nullptr) {
            return a;
        }
        a.get_unique_id = reinterpret_cast<decltype(a.get_unique_id)>(dlsym(lib, "ncclGetUniqueId"));
        a.comm_init_rank = reinterpret_cast<decltype(a.comm_init_rank)>(dlsym(lib, "ncclCommInitRank"));
        a.all_reduce = reinterpret_cast<decltype(a.all_reduce)>(dlsym(lib, "ncclAllReduce"));
        a.comm_destroy = reinterpret_cast<decltype(a.comm_destroy)>(dlsym(lib, "ncclCommDestroy"));
        a.error_string = reinterpret_cast<decltype(a.error_string)>(dlsym(lib, "ncclGetErrorString"));
        a.ok = a.get_unique_id && a.comm_init_rank && a.all_reduce && a.comm_destroy && a.error_string;
        return a;
    }();
    return api;
}

void nccl_check(ncclResult_t rc, const char *what) {
    if (rc != ncclSuccess) {
        fail(LLAISYS_E_DEVICE, std::string(what) + ": " + nccl_api().error_string(rc));
    }
}

static_assert(sizeof(ncclUniqueId) == kUniqueIdBytes, "NCCL unique id size");

class NcclCollective final : public Collective {
public:
    NcclCollective(const void *unique_id, int rank, int world) : Collective(rank, world) {
        ncclUniqueId id;
        memcpy(&id, unique_id, sizeof(id));
        nccl_check(nccl_api().comm_init_rank(&_comm, world, id, rank), "ncclCommInitRank");
    }
    ~NcclCollective() override {
        if (_comm != nullptr) {
            nccl_api().comm_destroy(_comm);
        }
    }
    void allReduceSum(void *buf, size_t count, llaisysDataType_t dtype, llaisysStream_t stream) override {
        ncclDataType_t t;
        switch (dtype) {
        case LLAISYS_DTYPE_F32:
            t = ncclFloat32;
            break;
        case LLAISYS_DTYPE_F16:
            t = ncclFloat16;
            break;
        case LLAISYS_DTYPE_BF16:
            t = ncclBfloat16;
            break;
        default:
            fail(LLAISYS_E_INVALID, "all-reduce: unsupported data type");
        }
        nccl_check(nccl_api().all_reduce(buf, buf, count, t, ncclSum, _comm, static_cast<cudaStream_t>(stream)),
                   "ncclAllReduce");
    }

private:
    ncclComm_t _comm = nullptr;
};
} // namespace

std::unique_ptr<Collective> Collective::nccl(const void *unique_id, int rank, int world) {
    if (unique_id == nullptr || world < 1 || rank < 0 || rank >= world) {
        fail(LLAISYS_E_INVALID, "collective: bad unique id, rank or world size");
    }
    if (!nccl_api().ok) {
        fail(LLAISYS_E_UNSUPPORTED, "collective: libnccl.so.2 was not found");
    }
    return std::make_unique<NcclCollective>(unique_id, rank, world);
}

void ncclUniqueIdBytes(void *out) {
    if (out == nullptr) {
        fail(LLAISYS_E_INVALID, "collective: null output");
    }
    if (!nccl_api().ok) {
        fail(LLAISYS_E_UNSUPPORTED, "collective: libnccl.so.2 was not found");
    }
    ncclUniqueId id;
    nccl_check(nccl_api().get_unique_id(&id), "ncclGetUniqueId");
    memcpy(out, &id, sizeof(id));
}

} // namespace llaisys::comm
