// Strided view over a shared storage block: dtype, shape, element strides and a byte offset
// (same model and accessor names as the reference: src/tensor/tensor.hpp:15-58).
#pragma once

#include "../core/core.hpp"

#include <string>
#include <vector>

namespace llaisys {

class Tensor;
using tensor_t = std::shared_ptr<Tensor>;

class Tensor {
public:
    // Contiguous row-major tensor on (device_type, device). A CPU tensor made while a device runtime is
    // current gets pinned host memory from that runtime (reference: src/tensor/tensor.cpp:29-31).
    static tensor_t create(const std::vector<size_t> &shape, llaisysDataType_t dtype,
                           llaisysDeviceType_t device_type = LLAISYS_DEVICE_CPU, int device = 0);

    std::byte *data() { return _storage->memory() + _offset; }
    const std::byte *data() const { return _storage->memory() + _offset; }
    size_t ndim() const { return _shape.size(); }
    const std::vector<size_t> &shape() const { return _shape; }
    const std::vector<ptrdiff_t> &strides() const { return _strides; }
    llaisysDataType_t dtype() const { return _dtype; }
    llaisysDeviceType_t deviceType() const { return _storage->deviceType(); }
    int deviceId() const { return _storage->deviceId(); }
    size_t numel() const;
    size_t elementSize() const;

    std::string info() const;
    void debug() const; // synchronises the device, prints info() and every element

    bool isContiguous() const;

    // Metadata-only transforms; the result shares this tensor's storage.
    tensor_t permute(const std::vector<size_t> &order) const;
    tensor_t slice(size_t dim, size_t start, size_t end) const;
    tensor_t view(const std::vector<size_t> &shape) const; // throws when the strides cannot express it

    void load(const void *host_src); // numel * elementSize bytes from host memory; tensor must be contiguous

    tensor_t contiguous() const;
    tensor_t reshape(const std::vector<size_t> &shape) const;
    tensor_t to(llaisysDeviceType_t device_type, int device = -1) const;

private:
    Tensor(llaisysDataType_t dtype, std::vector<size_t> shape, std::vector<ptrdiff_t> strides,
           core::storage_t storage, size_t offset_bytes)
        : _dtype(dtype), _shape(std::move(shape)), _strides(std::move(strides)), _storage(std::move(storage)),
          _offset(offset_bytes) {}

    llaisysDataType_t _dtype;
    std::vector<size_t> _shape;
    std::vector<ptrdiff_t> _strides; // in elements
    core::storage_t _storage;
    size_t _offset; // in bytes
};

// Strided element copy between two tensors of equal shape and dtype on one device (used by contiguous()
// and by the rearrange operator).
void copy_strided(Tensor &dst, const Tensor &src);

} // namespace llaisys
