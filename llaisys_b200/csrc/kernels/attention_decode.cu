#include "device_utils.cuh"
#include "kernels.hpp"
namespace llaisys::kernels {
int attention_decode_split(stream_t, llaisysDataType_t, const KVView &, const AttnBatch &, const void *, float,
                           const AttnOut &, const AttnScratch &) { return -1; }
void attention_decode_split_scratch(int32_t, int32_t, int32_t, int32_t, int32_t, size_t *partials_floats,
                                    size_t *counters_len) { *partials_floats = 0; *counters_len = 0; }
}
