// Per-thread device context: which device is current, its stream, and where tensor memory comes from.
//
// Shape of the design is the reference's (src/core/context/context.cpp:7-77, src/core/runtime/runtime.cpp:7-71,
// src/core/storage/storage.cpp:6-39): a thread_local Context owns one Runtime per (device type, device id);
// a Runtime owns one stream and one allocator; a Storage is a ref-counted block that returns to its Runtime
// when the last tensor using it goes away. Three behaviours differ on purpose:
//   * Runtimes are created on first use for ANY device id and are kept (the reference copies its runtime
//     vector in setDevice, so a lazily created Runtime -- and its stream -- is rebuilt on every switch);
//   * teardown deletes each Runtime exactly once;
//   * device blocks are cached and reused (the reference calls the device allocator for every tensor), which
//     on CUDA avoids a device-wide synchronising cudaFree per temporary.
#pragma once

#include "llaisys.h"
#include "llaisys/runtime.h"

#include <cstddef>
#include <map>
#include <memory>
#include <vector>

namespace llaisys::core {

class Runtime;
class Storage;
using storage_t = std::shared_ptr<Storage>;

// Size-bucketed cache in front of the device allocator. All users of a Runtime queue work on its single
// stream, so a block freed by one tensor can be handed to the next without waiting for the device.
class BlockCache {
public:
    explicit BlockCache(const LlaisysRuntimeAPI *api) : _api(api) {}
    ~BlockCache();
    BlockCache(const BlockCache &) = delete;
    BlockCache &operator=(const BlockCache &) = delete;

    std::byte *allocate(size_t bytes);
    void release(std::byte *ptr);
    void trim(); // hand every cached block back to the device
    size_t cachedBytes() const { return _cached_bytes; }

private:
    static size_t roundUp(size_t bytes);
    const LlaisysRuntimeAPI *_api;
    std::multimap<size_t, std::byte *> _free;  // rounded size -> block
    std::map<std::byte *, size_t> _live;       // block -> rounded size
    size_t _cached_bytes = 0;
};

class Runtime : public std::enable_shared_from_this<Runtime> {
public:
    Runtime(llaisysDeviceType_t device_type, int device_id);
    ~Runtime();
    Runtime(const Runtime &) = delete;
    Runtime &operator=(const Runtime &) = delete;

    llaisysDeviceType_t deviceType() const { return _device_type; }
    int deviceId() const { return _device_id; }
    const LlaisysRuntimeAPI *api() const { return _api; }
    llaisysStream_t stream() const { return _stream; }
    void synchronize() const { _api->stream_synchronize(_stream); }
    void activate() const { _api->set_device(_device_id); }

    storage_t allocateDeviceStorage(size_t bytes);
    storage_t allocateHostStorage(size_t bytes); // pinned on CUDA runtimes
    void freeStorage(Storage *storage);

private:
    llaisysDeviceType_t _device_type;
    int _device_id;
    const LlaisysRuntimeAPI *_api;
    llaisysStream_t _stream;
    BlockCache _cache;
};

class Storage {
public:
    Storage(std::byte *memory, size_t bytes, std::shared_ptr<Runtime> runtime, bool is_host)
        : _memory(memory), _size(bytes), _runtime(std::move(runtime)), _is_host(is_host) {}
    ~Storage() { _runtime->freeStorage(this); }
    Storage(const Storage &) = delete;
    Storage &operator=(const Storage &) = delete;

    std::byte *memory() const { return _memory; }
    size_t size() const { return _size; }
    bool isHost() const { return _is_host; }
    // Host-side staging blocks of a device runtime count as CPU memory, device 0.
    llaisysDeviceType_t deviceType() const { return _is_host ? LLAISYS_DEVICE_CPU : _runtime->deviceType(); }
    int deviceId() const { return _is_host ? 0 : _runtime->deviceId(); }

private:
    std::byte *_memory;
    size_t _size;
    std::shared_ptr<Runtime> _runtime; // a block keeps its runtime (stream, cache) alive
    bool _is_host;
};

class Context {
public:
    ~Context();
    Context(const Context &) = delete;
    Context &operator=(const Context &) = delete;

    // Makes the device current for this thread (no-op if it already is); throws on an id the device type
    // does not have.
    void setDevice(llaisysDeviceType_t device_type, int device_id);
    Runtime &runtime();

    friend Context &context();

private:
    Context();
    std::vector<std::shared_ptr<Runtime>> _runtimes[LLAISYS_DEVICE_TYPE_COUNT];
    Runtime *_current = nullptr;
};

// The calling thread's context. On first use it activates device 0 of the first non-CPU device type that
// has devices, else the CPU (reference: src/core/context/context.cpp:7-32).
Context &context();

} // namespace llaisys::core
