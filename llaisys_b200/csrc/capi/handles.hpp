// The opaque tensor handle of the C ABI: a heap object holding one reference to a tensor
// (reference: src/llaisys/llaisys_tensor.hpp:7-9).
#pragma once

#include "../tensor/tensor.hpp"

struct LlaisysTensor {
    llaisys::tensor_t tensor;
};
