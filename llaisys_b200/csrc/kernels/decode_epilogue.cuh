// Last-arriver side of the split-KV combine, shared by the decode kernels.
//
// A (sequence, kv-head) pair that was cut across E CTAs leaves E partial results, slot i holding for every head
// h of the group the un-normalised output o_i,h[128] relative to its own max m_i,h (log2 units) and sum l_i,h:
//     float [E][group][130]   (o[128], m, l)
// The CTA whose arrival completes the pair merges them:  M = max_i m_i,  w_i = 2^(m_i - M),
//     out = sum_i w_i o_i / sum_i w_i l_i.
// Latency matters more than arithmetic here (each dependent L2 read costs ~0.5 us and the merge sits on the
// kernel's critical path), so the loads are batched: all (m, l) of up to 256 parts are staged in shared memory
// in one round trip, then every thread (one output dimension each) accumulates o with 4 parts x `group` heads of
// independent loads in flight. More than 256 parts are folded in chunks with a running (M, L, O).
#pragma once

#include "mma_utils.cuh"

namespace llaisys::kernels {

constexpr int kCombineChunk = 256; // parts staged per round; needs 2 * kCombineChunk * group floats of staging

// All `n_threads` (== 128 == head_dim) threads of the merging group call this; `sync` is their barrier.
// stage: shared memory, at least 2 * kCombineChunk * group floats. out_row0: index of head 0's output row.
template <bool kBf16, typename Sync>
__device__ __forceinline__ void combine_partials(const float *first, int expected, int group, int tid, float *stage,
                                                 Sync sync, void *out, float *part, long long out_row0) {
    constexpr int kD = 128, kMaxGroup = 8, kStride = kD + 2;
    float m_run[kMaxGroup], l_run[kMaxGroup], o_run[kMaxGroup];
#pragma unroll
    for (int h = 0; h < kMaxGroup; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
        o_run[h] = 0.f;
    }
    float *m_s = stage, *l_s = stage + kCombineChunk * group;
    for (int c0 = 0; c0 < expected; c0 += kCombineChunk) {
        const int ce = min(kCombineChunk, expected - c0);
        sync(); // staging area free (previous chunk, or the caller's last use)
        for (int idx = tid; idx < ce * group; idx += kD) {
            const float *pp = first + (long long)(c0 * group + idx) * kStride;
            m_s[idx] = __ldcg(pp + kD);
            l_s[idx] = __ldcg(pp + kD + 1);
        }
        sync();
        // fold this chunk's maxima into the running ones
#pragma unroll
        for (int h = 0; h < kMaxGroup; ++h) {
            if (h < group) {
                float cm = -INFINITY;
                for (int i = 0; i < ce; ++i) {
                    cm = fmaxf(cm, m_s[i * group + h]);
                }
                const float nm = fmaxf(m_run[h], cm);
                const float sc = (m_run[h] == -INFINITY) ? 0.f : fast_exp2(m_run[h] - nm);
                l_run[h] *= sc;
                o_run[h] *= sc;
                m_run[h] = nm;
            }
        }
        // accumulate: 4 parts x group heads of independent loads per round
        for (int i0 = 0; i0 < ce; i0 += 4) {
            float v[4][kMaxGroup];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int h = 0; h < kMaxGroup; ++h) {
                    v[u][h] = (i0 + u < ce && h < group)
                                  ? __ldcg(first + (long long)((c0 + i0 + u) * group + h) * kStride + tid)
                                  : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int h = 0; h < kMaxGroup; ++h) {
                    if (i0 + u < ce && h < group) {
                        const float mi = m_s[(i0 + u) * group + h];
                        const float w = (mi == -INFINITY) ? 0.f : fast_exp2(mi - m_run[h]);
                        l_run[h] = fmaf(l_s[(i0 + u) * group + h], w, l_run[h]);
                        o_run[h] = fmaf(v[u][h], w, o_run[h]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < kMaxGroup; ++h) {
        if (h < group) {
            const long long row = out_row0 + h;
            const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
            if (part != nullptr) {
                part[row * kStride + tid] = o_run[h] * inv;
                if (tid == 0) {
                    part[row * kStride + kD] = m_run[h] * 0.6931471805599453f; // log2 units -> natural log
                    part[row * kStride + kD + 1] = l_run[h];
                }
            } else {
                store_out<kBf16>(out, row * kD + tid, o_run[h] * inv);
            }
        }
    }
}


// Warp edition for partials laid out float [E][group][132] (o[128], m, l, 2 pad: 16-byte aligned rows): lane j owns
// output dimensions 4j .. 4j+3 of every head. A dependent read of another SM's freshly written partial costs about
// a microsecond, so a round keeps kParts parts x kHeads heads of 16-byte loads in flight per lane (the common cut,
// 2-4 pieces per pair, merges in ONE round trip); the (m, l) scalars of a round are loaded one per lane and
// broadcast with shuffles instead of occupying kParts * kHeads more registers.
template <bool kBf16, int kHeads, int kParts>
__device__ __forceinline__ void warp_combine_impl(const float *first, int expected, int group, int lane, void *out,
                                                  float *part, long long out_row0) {
    constexpr int kD = 128, kStride = kD + 4, kOutStride = kD + 2;
    static_assert(kHeads * kParts <= 32, "one (m, l) pair per lane per round");
    float m_run[kHeads], l_run[kHeads];
    float4 o_run[kHeads];
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
        o_run[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int i0 = 0; i0 < expected; i0 += kParts) {
        float4 v[kParts][kHeads];
#pragma unroll
        for (int u = 0; u < kParts; ++u) {
#pragma unroll
            for (int h = 0; h < kHeads; ++h) {
                v[u][h] = (i0 + u < expected && h < group)
                              ? __ldcg(reinterpret_cast<const float4 *>(first + (long long)((i0 + u) * group + h) * kStride) + lane)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        // lane u * kHeads + h fetches (m, l) of part i0 + u, head h
        float2 ml = make_float2(-INFINITY, 0.f);
        {
            const int u = lane / kHeads, h = lane - u * kHeads;
            if (u < kParts && i0 + u < expected && h < group) {
                ml = __ldcg(reinterpret_cast<const float2 *>(first + (long long)((i0 + u) * group + h) * kStride + kD));
            }
        }
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            float mi[kParts], li[kParts];
            float nm = m_run[h];
#pragma unroll
            for (int u = 0; u < kParts; ++u) {
                mi[u] = __shfl_sync(0xffffffffu, ml.x, u * kHeads + h);
                li[u] = __shfl_sync(0xffffffffu, ml.y, u * kHeads + h);
                nm = fmaxf(nm, mi[u]);
            }
            const float ref = nm == -INFINITY ? 0.f : nm;
            const float sc = fast_exp2(m_run[h] - ref); // 2^(-inf) = 0 on the first round
            l_run[h] *= sc;
            o_run[h].x *= sc;
            o_run[h].y *= sc;
            o_run[h].z *= sc;
            o_run[h].w *= sc;
#pragma unroll
            for (int u = 0; u < kParts; ++u) {
                const float w = fast_exp2(mi[u] - ref);
                l_run[h] = fmaf(li[u], w, l_run[h]);
                o_run[h].x = fmaf(v[u][h].x, w, o_run[h].x);
                o_run[h].y = fmaf(v[u][h].y, w, o_run[h].y);
                o_run[h].z = fmaf(v[u][h].z, w, o_run[h].z);
                o_run[h].w = fmaf(v[u][h].w, w, o_run[h].w);
            }
            m_run[h] = nm;
        }
    }
    __syncwarp(); // every lane has consumed its loads: `part` may lie over the partials just read
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
        if (h < group) {
            const long long row = out_row0 + h;
            const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
            const float r[4] = {o_run[h].x * inv, o_run[h].y * inv, o_run[h].z * inv, o_run[h].w * inv};
            if (part != nullptr) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    part[row * kOutStride + lane * 4 + e] = r[e];
                }
                if (lane == 0) {
                    part[row * kOutStride + kD] = m_run[h] * 0.6931471805599453f; // log2 units -> natural log
                    part[row * kOutStride + kD + 1] = l_run[h];
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    store_out<kBf16>(out, row * kD + lane * 4 + e, r[e]);
                }
            }
        }
    }
}

template <bool kBf16>
__device__ __forceinline__ void warp_combine_partials(const float *first, int expected, int group, int lane, void *out,
                                                      float *part, long long out_row0) {
    if (group <= 4) {
        warp_combine_impl<kBf16, 4, 4>(first, expected, group, lane, out, part, out_row0);
    } else if (group <= 6) {
        warp_combine_impl<kBf16, 6, 4>(first, expected, group, lane, out, part, out_row0);
    } else {
        warp_combine_impl<kBf16, 8, 2>(first, expected, group, lane, out, part, out_row0);
    }
}

// The same merge as a function of its own, for kernels in which the inlined loop does not come out well: it keeps up
// to 96 registers of loads in flight, and inlined into the exchange instantiation of the TMA decode kernel (whose other
// warps sit at the register limit) it ran 2.3 times slower than in the ordinary one. Compiled by itself it does not
// depend on its surroundings; the call costs about a microsecond, which is why the ordinary kernel keeps the inlined one.
template <bool kBf16>
__device__ __noinline__ void warp_combine_partials_call(const float *first, int expected, int group, int lane, void *out,
                                                        float *part, long long out_row0) {
    warp_combine_partials<kBf16>(first, expected, group, lane, out, part, out_row0);
}

} // namespace llaisys::kernels
