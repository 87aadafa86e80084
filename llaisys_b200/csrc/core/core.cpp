#include "core.hpp"

#include "../common/check.hpp"
#include "../device/runtime_api.hpp"

namespace llaisys::core {

// ---- BlockCache ---------------------------------------------------------------------------------

size_t BlockCache::roundUp(size_t bytes) {
    // 512 B granularity up to 1 MiB, then 2 MiB granularity: few distinct sizes, little slack.
    constexpr size_t kSmall = 512, kLarge = size_t(2) << 20;
    if (bytes == 0) {
        bytes = 1;
    }
    const size_t g = bytes <= (size_t(1) << 20) ? kSmall : kLarge;
    return (bytes + g - 1) / g * g;
}

std::byte *BlockCache::allocate(size_t bytes) {
    const size_t want = roundUp(bytes);
    auto it = _free.find(want);
    std::byte *block;
    if (it != _free.end()) {
        block = it->second;
        _free.erase(it);
        _cached_bytes -= want;
    } else {
        block = static_cast<std::byte *>(_api->malloc_device(want));
        if (block == nullptr) {
            trim();
            block = static_cast<std::byte *>(_api->malloc_device(want));
        }
        ASSERT(block != nullptr, "device allocation of " << want << " bytes failed");
    }
    _live.emplace(block, want);
    return block;
}

void BlockCache::release(std::byte *ptr) {
    auto it = _live.find(ptr);
    ASSERT(it != _live.end(), "release of a block this runtime did not allocate");
    _free.emplace(it->second, ptr);
    _cached_bytes += it->second;
    _live.erase(it);
}

void BlockCache::trim() {
    for (auto &e : _free) {
        _api->free_device(e.second);
    }
    _free.clear();
    _cached_bytes = 0;
}

BlockCache::~BlockCache() {
    trim(); // _live is empty here: every Storage holds a reference to its Runtime
}

// ---- Runtime ------------------------------------------------------------------------------------

Runtime::Runtime(llaisysDeviceType_t device_type, int device_id)
    : _device_type(device_type), _device_id(device_id), _api(device::getRuntimeAPI(device_type)), _stream(nullptr),
      _cache(_api) {
    _api->set_device(_device_id);
    _stream = _api->create_stream();
}

Runtime::~Runtime() {
    // Neither freeing device memory nor destroying a stream needs the device to be current, so the
    // destructor leaves the thread's current device alone.
    _cache.trim();
    _api->destroy_stream(_stream);
}

storage_t Runtime::allocateDeviceStorage(size_t bytes) {
    return std::make_shared<Storage>(_cache.allocate(bytes), bytes, shared_from_this(), false);
}

storage_t Runtime::allocateHostStorage(size_t bytes) {
    return std::make_shared<Storage>(static_cast<std::byte *>(_api->malloc_host(bytes)), bytes, shared_from_this(), true);
}

void Runtime::freeStorage(Storage *storage) {
    if (storage->isHost()) {
        _api->free_host(storage->memory());
    } else {
        _cache.release(storage->memory());
    }
}

// ---- Context ------------------------------------------------------------------------------------

Context::Context() {
    for (int t = 1; t < LLAISYS_DEVICE_TYPE_COUNT && _current == nullptr; ++t) {
        const auto type = static_cast<llaisysDeviceType_t>(t);
        if (device::getRuntimeAPI(type)->get_device_count() > 0) {
            setDevice(type, 0);
        }
    }
    if (_current == nullptr) {
        setDevice(LLAISYS_DEVICE_CPU, 0);
    }
}

Context::~Context() {
    _current = nullptr;
    for (auto &per_type : _runtimes) {
        per_type.clear();
    }
}

void Context::setDevice(llaisysDeviceType_t device_type, int device_id) {
    if (_current != nullptr && _current->deviceType() == device_type && _current->deviceId() == device_id) {
        return;
    }
    CHECK_ARGUMENT(device_type >= 0 && device_type < LLAISYS_DEVICE_TYPE_COUNT, "invalid device type");
    auto &slots = _runtimes[device_type];
    if (slots.empty()) {
        const int n = device::getRuntimeAPI(device_type)->get_device_count();
        slots.resize(n > 0 ? size_t(n) : 0);
    }
    CHECK_ARGUMENT(device_id >= 0 && size_t(device_id) < slots.size(), "invalid device id");
    if (!slots[device_id]) {
        slots[device_id] = std::make_shared<Runtime>(device_type, device_id);
    }
    slots[device_id]->activate();
    _current = slots[device_id].get();
}

Runtime &Context::runtime() {
    ASSERT(_current != nullptr, "no runtime is active; call setDevice() first");
    return *_current;
}

Context &context() {
    thread_local Context ctx;
    return ctx;
}

} // namespace llaisys::core
