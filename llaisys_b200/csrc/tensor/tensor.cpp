#include "tensor.hpp"

#include "../common/check.hpp"
#include "../common/dtypes.hpp"
#include "../ops/ops.hpp"

#include <algorithm>
#include <cstring>
#include <iostream>
#include <sstream>

namespace llaisys {

namespace {

std::vector<ptrdiff_t> row_major_strides(const std::vector<size_t> &shape) {
    std::vector<ptrdiff_t> strides(shape.size());
    ptrdiff_t run = 1;
    for (size_t i = shape.size(); i-- > 0;) {
        strides[i] = run;
        run *= ptrdiff_t(shape[i]);
    }
    return strides;
}

size_t product(const std::vector<size_t> &shape) {
    size_t n = 1;
    for (size_t s : shape) {
        n *= s;
    }
    return n;
}

template <typename T>
void print_rec(const T *p, const std::vector<size_t> &shape, const std::vector<ptrdiff_t> &strides, size_t dim) {
    if (shape.empty()) {
        return;
    }
    if (dim + 1 == shape.size()) {
        for (size_t i = 0; i < shape[dim]; ++i) {
            const T &e = p[ptrdiff_t(i) * strides[dim]];
            if constexpr (std::is_same_v<T, bf16_t> || std::is_same_v<T, fp16_t>) {
                std::cout << utils::cast<float>(e) << " ";
            } else if constexpr (sizeof(T) == 1) {
                std::cout << int(e) << " ";
            } else {
                std::cout << e << " ";
            }
        }
        std::cout << std::endl;
        return;
    }
    for (size_t i = 0; i < shape[dim]; ++i) {
        print_rec(p + ptrdiff_t(i) * strides[dim], shape, strides, dim + 1);
    }
}

void print_any(const std::byte *p, llaisysDataType_t dtype, const std::vector<size_t> &shape,
               const std::vector<ptrdiff_t> &strides) {
#define LLAISYS_PRINT_CASE(TAG, T) \
    case TAG:                      \
        return print_rec(reinterpret_cast<const T *>(p), shape, strides, 0)
    switch (dtype) {
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_BYTE, uint8_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_BOOL, uint8_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_I8, int8_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_I16, int16_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_I32, int32_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_I64, int64_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_U8, uint8_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_U16, uint16_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_U32, uint32_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_U64, uint64_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_F16, fp16_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_BF16, bf16_t);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_F32, float);
        LLAISYS_PRINT_CASE(LLAISYS_DTYPE_F64, double);
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
#undef LLAISYS_PRINT_CASE
}

} // namespace

tensor_t Tensor::create(const std::vector<size_t> &shape, llaisysDataType_t dtype, llaisysDeviceType_t device_type,
                        int device) {
    const size_t bytes = product(shape) * utils::dsize(dtype);
    auto &ctx = core::context();
    core::storage_t storage;
    if (device_type == LLAISYS_DEVICE_CPU && ctx.runtime().deviceType() != LLAISYS_DEVICE_CPU) {
        storage = ctx.runtime().allocateHostStorage(bytes);
    } else {
        ctx.setDevice(device_type, device);
        storage = ctx.runtime().allocateDeviceStorage(bytes);
    }
    return tensor_t(new Tensor(dtype, shape, row_major_strides(shape), std::move(storage), 0));
}

size_t Tensor::numel() const { return product(_shape); }
size_t Tensor::elementSize() const { return utils::dsize(_dtype); }

std::string Tensor::info() const {
    std::ostringstream os;
    os << "Tensor: shape[ ";
    for (size_t s : _shape) {
        os << s << " ";
    }
    os << "] strides[ ";
    for (ptrdiff_t s : _strides) {
        os << s << " ";
    }
    os << "] dtype=" << _dtype;
    return os.str();
}

void Tensor::debug() const {
    auto &ctx = core::context();
    ctx.setDevice(deviceType(), deviceId());
    ctx.runtime().api()->device_synchronize();
    std::cout << info() << std::endl;
    if (deviceType() == LLAISYS_DEVICE_CPU) {
        print_any(data(), _dtype, _shape, _strides);
        return;
    }
    // Copy the smallest span of storage that covers every element of this view, then print with the
    // view's own strides.
    size_t span = 1;
    for (size_t i = 0; i < _shape.size(); ++i) {
        if (_shape[i] == 0) {
            return;
        }
        span += (_shape[i] - 1) * size_t(_strides[i]);
    }
    std::vector<std::byte> host(span * elementSize());
    ctx.runtime().api()->memcpy_sync(host.data(), data(), host.size(), LLAISYS_MEMCPY_D2H);
    print_any(host.data(), _dtype, _shape, _strides);
}

bool Tensor::isContiguous() const {
    ptrdiff_t expect = 1;
    for (size_t i = _shape.size(); i-- > 0;) {
        if (_shape[i] != 1 && _strides[i] != expect) {
            return false;
        }
        expect *= ptrdiff_t(_shape[i]);
    }
    return true;
}

tensor_t Tensor::permute(const std::vector<size_t> &order) const {
    CHECK_ARGUMENT(order.size() == ndim(), "permute: order must name every dimension");
    std::vector<bool> seen(ndim(), false);
    std::vector<size_t> shape(ndim());
    std::vector<ptrdiff_t> strides(ndim());
    for (size_t i = 0; i < ndim(); ++i) {
        CHECK_ARGUMENT(order[i] < ndim() && !seen[order[i]], "permute: order is not a permutation");
        seen[order[i]] = true;
        shape[i] = _shape[order[i]];
        strides[i] = _strides[order[i]];
    }
    return tensor_t(new Tensor(_dtype, std::move(shape), std::move(strides), _storage, _offset));
}

tensor_t Tensor::slice(size_t dim, size_t start, size_t end) const {
    CHECK_ARGUMENT(dim < ndim(), "slice: dimension out of range");
    CHECK_ARGUMENT(start <= end && end <= _shape[dim], "slice: range out of bounds");
    std::vector<size_t> shape = _shape;
    shape[dim] = end - start;
    const size_t offset = _offset + start * size_t(_strides[dim]) * elementSize();
    return tensor_t(new Tensor(_dtype, std::move(shape), _strides, _storage, offset));
}

// A view exists iff every maximal run of old dimensions that is laid out like one dense block can be cut
// into whole new dimensions. Walk the old shape from the right, closing a block wherever the next stride
// does not continue it, and hand out new dimensions (also from the right) until they fill the block.
tensor_t Tensor::view(const std::vector<size_t> &shape) const {
    CHECK_ARGUMENT(product(shape) == numel(), "view: element count differs");
    if (numel() == 0 || ndim() == 0) {
        return tensor_t(new Tensor(_dtype, shape, row_major_strides(shape), _storage, _offset));
    }
    std::vector<ptrdiff_t> strides(shape.size(), 1);
    ptrdiff_t next_new = ptrdiff_t(shape.size()) - 1;
    ptrdiff_t block_stride = _strides.back();
    size_t block_elems = 1, handed_out = 1;
    for (size_t d = ndim(); d-- > 0;) {
        block_elems *= _shape[d];
        const bool block_ends =
            d == 0 || (_shape[d - 1] != 1 && _strides[d - 1] != ptrdiff_t(block_elems) * block_stride);
        if (!block_ends) {
            continue;
        }
        while (next_new >= 0 && (handed_out < block_elems || shape[next_new] == 1)) {
            strides[next_new] = ptrdiff_t(handed_out) * block_stride;
            handed_out *= shape[next_new];
            --next_new;
        }
        CHECK_ARGUMENT(handed_out == block_elems, "view: tensor layout cannot be viewed with this shape");
        if (d > 0) {
            block_stride = _strides[d - 1];
            block_elems = 1;
            handed_out = 1;
        }
    }
    CHECK_ARGUMENT(next_new < 0, "view: shapes are incompatible");
    return tensor_t(new Tensor(_dtype, shape, std::move(strides), _storage, _offset));
}

void Tensor::load(const void *host_src) {
    ASSERT(isContiguous(), "load: destination tensor must be contiguous");
    auto &ctx = core::context();
    const size_t bytes = numel() * elementSize();
    if (deviceType() == LLAISYS_DEVICE_CPU) {
        std::memcpy(data(), host_src, bytes);
        return;
    }
    ctx.setDevice(deviceType(), deviceId());
    ctx.runtime().api()->memcpy_sync(data(), host_src, bytes, LLAISYS_MEMCPY_H2D);
}

void copy_strided(Tensor &dst, const Tensor &src) { ops::rearrange_raw(dst, src); }

tensor_t Tensor::contiguous() const {
    if (isContiguous()) {
        return tensor_t(new Tensor(_dtype, _shape, _strides, _storage, _offset));
    }
    tensor_t out = create(_shape, _dtype, deviceType(), deviceId());
    copy_strided(*out, *this);
    return out;
}

tensor_t Tensor::reshape(const std::vector<size_t> &shape) const { return contiguous()->view(shape); }

tensor_t Tensor::to(llaisysDeviceType_t device_type, int device) const {
    if (device < 0) {
        device = (device_type == deviceType()) ? deviceId() : 0;
    }
    tensor_t src = contiguous();
    tensor_t out = create(_shape, _dtype, device_type, device);
    const size_t bytes = numel() * elementSize();
    auto &ctx = core::context();
    if (device_type == LLAISYS_DEVICE_CPU && deviceType() == LLAISYS_DEVICE_CPU) {
        std::memcpy(out->data(), src->data(), bytes);
    } else if (device_type == LLAISYS_DEVICE_CPU) {
        ctx.setDevice(deviceType(), deviceId());
        ctx.runtime().api()->memcpy_sync(out->data(), src->data(), bytes, LLAISYS_MEMCPY_D2H);
    } else {
        ctx.setDevice(device_type, device);
        const auto kind = deviceType() == LLAISYS_DEVICE_CPU ? LLAISYS_MEMCPY_H2D : LLAISYS_MEMCPY_D2D;
        ctx.runtime().api()->memcpy_sync(out->data(), src->data(), bytes, kind);
    }
    return out;
}

} // namespace llaisys
