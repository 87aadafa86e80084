// Error reporting for the legacy (void-returning) part of the ABI.
//
// Convention kept from the reference (src/utils/check.hpp:4-44): a violated precondition prints one
// "[ERROR] ... from <function> at <file>:<line>." line to stderr and throws; nothing catches the
// exception before the extern "C" frame, so the process ends. The status-returning entry points of
// the paged-KV API catch at the boundary instead (see capi/paged_kv.cc).
#pragma once

#include <sstream>
#include <stdexcept>
#include <string>

#include "llaisys.h"

namespace llaisys::utils {
const char *dtype_to_str(llaisysDataType_t dtype);
}

namespace llaisys::detail {

[[noreturn]] void raise(const char *kind, const std::string &what, const char *func, const char *file, int line,
                        bool invalid_argument);

} // namespace llaisys::detail

#define LLAISYS_RAISE_(kind, msg_expr, is_invalid)                                                          \
    do {                                                                                                    \
        std::ostringstream os___;                                                                           \
        os___ << msg_expr;                                                                                  \
        ::llaisys::detail::raise(kind, os___.str(), __func__, __FILE__, __LINE__, is_invalid);              \
    } while (0)

// Same spellings as the reference so operator code reads the same way.
#define EXCEPTION_UNSUPPORTED_DEVICE LLAISYS_RAISE_("Unsupported device", "", false)
#define EXCEPTION_UNSUPPORTED_DATATYPE(DT__) \
    LLAISYS_RAISE_("Unsupported data type", ::llaisys::utils::dtype_to_str(DT__), false)
#define TO_BE_IMPLEMENTED() LLAISYS_RAISE_("Unimplemented function", "", false)
#define EXCEPTION_SHAPE_MISMATCH LLAISYS_RAISE_("Shapes mismatch", "", true)
#define EXCEPTION_DATATYPE_MISMATCH LLAISYS_RAISE_("Datatypes mismatch", "", true)
#define EXCEPTION_DEVICE_MISMATCH LLAISYS_RAISE_("Device mismatch", "input tensors must be on the same device", false)

#define CHECK_ARGUMENT(cond, msg)                          \
    do {                                                   \
        if (!(cond)) {                                     \
            LLAISYS_RAISE_("Invalid argument", msg, true); \
        }                                                  \
    } while (0)

#define ASSERT(cond, msg)                                                   \
    do {                                                                    \
        if (!(cond)) {                                                      \
            LLAISYS_RAISE_("Assertion failed", msg << " [" #cond "]", false); \
        }                                                                   \
    } while (0)

#define CHECK_SAME_SHAPE(FIRST, ...)                 \
    do {                                             \
        for (const auto &other___ : {__VA_ARGS__}) { \
            if (!((FIRST) == other___)) {            \
                EXCEPTION_SHAPE_MISMATCH;            \
            }                                        \
        }                                            \
    } while (0)

#define CHECK_SAME_DTYPE(FIRST, ...)                 \
    do {                                             \
        for (const auto &other___ : {__VA_ARGS__}) { \
            if ((FIRST) != other___) {               \
                EXCEPTION_DATATYPE_MISMATCH;         \
            }                                        \
        }                                            \
    } while (0)

#define CHECK_SAME_DEVICE(FIRST, ...)                                                                         \
    do {                                                                                                      \
        for (const auto &t___ : {__VA_ARGS__}) {                                                              \
            if ((FIRST)->deviceType() != t___->deviceType() || (FIRST)->deviceId() != t___->deviceId()) {     \
                EXCEPTION_DEVICE_MISMATCH;                                                                    \
            }                                                                                                 \
        }                                                                                                     \
    } while (0)
