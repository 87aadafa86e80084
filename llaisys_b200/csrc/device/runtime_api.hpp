// One table of twelve entry points per device type (C layout in include/llaisys/runtime.h).
#pragma once

#include "llaisys/runtime.h"

namespace llaisys::device {

// Table for a device type; a type this build cannot drive gets the "absent" table, which reports
// zero devices and throws from every other entry (reference: src/device/runtime_api.cpp:5-88).
const LlaisysRuntimeAPI *getRuntimeAPI(llaisysDeviceType_t device_type);
const LlaisysRuntimeAPI *getUnsupportedRuntimeAPI();

namespace cpu {
const LlaisysRuntimeAPI *getRuntimeAPI();
}

#ifdef ENABLE_NVIDIA_API
namespace nvidia {
const LlaisysRuntimeAPI *getRuntimeAPI();
}
#endif

} // namespace llaisys::device
