#include "collective.hpp"

#include "../kv/paged_kv.hpp"
#include "llaisys/paged_kv.h"

#include <string>

namespace llaisys::comm {

namespace {

[[noreturn]] void fail(int code, const std::string &msg) { throw kv::StatusError(code, msg); }

class CallbackCollective final : public Collective {
public:
    CallbackCollective(AllReduceCallback fn, void *user, int rank, int world) : Collective(rank, world), _fn(fn), _user(user) {}
    void allReduceSum(void *buf, size_t count, llaisysDataType_t dtype, llaisysStream_t) override {
        const int rc = _fn(buf, count, int(dtype), _user);
        if (rc != 0) {
            fail(LLAISYS_E_DEVICE, "all-reduce callback failed with code " + std::to_string(rc));
        }
    }

private:
    AllReduceCallback _fn;
    void *_user;
};

} // namespace

std::unique_ptr<Collective> Collective::callback(AllReduceCallback fn, void *user, int rank, int world) {
    if (fn == nullptr || world < 1 || rank < 0 || rank >= world) {
        fail(LLAISYS_E_INVALID, "collective: bad callback, rank or world size");
    }
    return std::make_unique<CallbackCollective>(fn, user, rank, world);
}

#ifndef ENABLE_NVIDIA_API
std::unique_ptr<Collective> Collective::nccl(const void *, int, int) {
    fail(LLAISYS_E_UNSUPPORTED, "this build has no NVIDIA backend");
}
void ncclUniqueIdBytes(void *) { fail(LLAISYS_E_UNSUPPORTED, "this build has no NVIDIA backend"); }
#endif

} // namespace llaisys::comm
