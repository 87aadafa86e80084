// The struct behind the opaque model handle of the C ABI, shared by the thunks that take one.
#pragma once

#include "../models/qwen2.hpp"

struct LlaisysQwen2Model {
    llaisys::models::Qwen2 impl;
    LlaisysQwen2Model(const LlaisysQwen2Meta &meta, llaisysDeviceType_t device, int device_id, int tp_rank = 0, int tp_world = 1)
        : impl(meta, device, device_id, tp_rank, tp_world) {}
};
