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
// The running state of a merge: per head the max m (log2 units), the sum l and this lane's four output dimensions.
template <int kHeads>
struct MergeState {
    float m[kHeads], l[kHeads];
    float4 o[kHeads];
    __device__ __forceinline__ void clear() {
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            m[h] = -INFINITY;
            l[h] = 0.f;
            o[h] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
};

// Folds parts begin, begin + step, ... (< expected) into `st`. kShared: the parts lie in shared memory (plain loads)
// instead of global memory (L2 loads).
template <int kHeads, int kParts, bool kShared>
__device__ __forceinline__ void warp_merge_parts(MergeState<kHeads> &st, const float *first, int expected, int begin,
                                                 int step, int group, int lane) {
    constexpr int kD = 128, kStride = kD + 4;
    static_assert(kHeads * kParts <= 32, "one (m, l) pair per lane per round");
    auto load4 = [](const float *p) {
        if constexpr (kShared) {
            return *reinterpret_cast<const float4 *>(p);
        } else {
            return __ldcg(reinterpret_cast<const float4 *>(p));
        }
    };
    auto load2 = [](const float *p) {
        if constexpr (kShared) {
            return *reinterpret_cast<const float2 *>(p);
        } else {
            return __ldcg(reinterpret_cast<const float2 *>(p));
        }
    };
    for (int i0 = begin; i0 < expected; i0 += kParts * step) {
        float4 v[kParts][kHeads];
#pragma unroll
        for (int u = 0; u < kParts; ++u) {
#pragma unroll
            for (int h = 0; h < kHeads; ++h) {
                v[u][h] = (i0 + u * step < expected && h < group)
                              ? load4(first + (long long)((i0 + u * step) * group + h) * kStride + lane * 4)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        // lane u * kHeads + h fetches (m, l) of part i0 + u * step, head h
        float2 ml = make_float2(-INFINITY, 0.f);
        {
            const int u = lane / kHeads, h = lane - u * kHeads;
            if (u < kParts && i0 + u * step < expected && h < group) {
                ml = load2(first + (long long)((i0 + u * step) * group + h) * kStride + kD);
            }
        }
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            float mi[kParts], li[kParts];
            float nm = st.m[h];
#pragma unroll
            for (int u = 0; u < kParts; ++u) {
                mi[u] = __shfl_sync(0xffffffffu, ml.x, u * kHeads + h);
                li[u] = __shfl_sync(0xffffffffu, ml.y, u * kHeads + h);
                nm = fmaxf(nm, mi[u]);
            }
            const float ref = nm == -INFINITY ? 0.f : nm;
            const float sc = fast_exp2(st.m[h] - ref); // 2^(-inf) = 0 on the first round
            st.l[h] *= sc;
            st.o[h].x *= sc;
            st.o[h].y *= sc;
            st.o[h].z *= sc;
            st.o[h].w *= sc;
#pragma unroll
            for (int u = 0; u < kParts; ++u) {
                const float w = fast_exp2(mi[u] - ref);
                st.l[h] = fmaf(li[u], w, st.l[h]);
                st.o[h].x = fmaf(v[u][h].x, w, st.o[h].x);
                st.o[h].y = fmaf(v[u][h].y, w, st.o[h].y);
                st.o[h].z = fmaf(v[u][h].z, w, st.o[h].z);
                st.o[h].w = fmaf(v[u][h].w, w, st.o[h].w);
            }
            st.m[h] = nm;
        }
    }
}

// Normalises a finished merge and stores it: rows of the K/V dtype into `out`, or (part != nullptr) rows of d + 2
// floats (o, m in natural-log units, l).
template <bool kBf16, int kHeads>
__device__ __forceinline__ void warp_merge_store(const MergeState<kHeads> &st, int group, int lane, void *out, float *part,
                                                 long long out_row0) {
    constexpr int kD = 128, kOutStride = kD + 2;
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
        if (h < group) {
            const long long row = out_row0 + h;
            const float inv = st.l[h] > 0.f ? 1.f / st.l[h] : 0.f;
            const float r[4] = {st.o[h].x * inv, st.o[h].y * inv, st.o[h].z * inv, st.o[h].w * inv};
            if (part != nullptr) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    part[row * kOutStride + lane * 4 + e] = r[e];
                }
                if (lane == 0) {
                    part[row * kOutStride + kD] = st.m[h] * 0.6931471805599453f; // log2 units -> natural log
                    part[row * kOutStride + kD + 1] = st.l[h];
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

// Leaves an unfinished merge as one more "part" (same layout as a partial result: o[128], m, l per head, rows of 132
// floats) at `dst`, shared or global memory: for merges that several warps share.
template <int kHeads>
__device__ __forceinline__ void warp_merge_stash(const MergeState<kHeads> &st, int group, int lane, float *dst) {
    constexpr int kD = 128, kStride = kD + 4;
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
        if (h < group) {
            *reinterpret_cast<float4 *>(dst + h * kStride + lane * 4) = st.o[h];
            if (lane == 0) {
                dst[h * kStride + kD] = st.m[h];
                dst[h * kStride + kD + 1] = st.l[h];
            }
        }
    }
}

template <bool kBf16, int kHeads, int kParts>
__device__ __forceinline__ void warp_combine_impl(const float *first, int expected, int group, int lane, void *out,
                                                  float *part, long long out_row0) {
    MergeState<kHeads> st;
    st.clear();
    warp_merge_parts<kHeads, kParts, false>(st, first, expected, 0, 1, group, lane);
    __syncwarp(); // every lane has consumed its loads: `part` may lie over the partials just read
    warp_merge_store<kBf16, kHeads>(st, group, lane, out, part, out_row0);
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

// A merge shared by n_warps warps of one CTA (for pairs cut into many pieces: one long sequence on a whole GPU leaves
// dozens of partials per pair, and one warp merges them four per round trip). Warp w folds parts w, w + n_warps, ...
// and leaves its unfinished state as part w of `stash` (global memory of the CTA's own, n_warps x group x 132 floats);
// after a barrier over the warps, one of them folds the n_warps stashed states and stores the result. Which warp takes which parts is
// fixed, so the bits do not depend on timing.
template <bool kBf16>
__device__ __forceinline__ void warp_merge_share(const float *first, int expected, int w, int n_warps, int group, int lane,
                                                 float *stash) {
    constexpr int kStride = 132;
    float *dst = stash + (long long)w * group * kStride;
    if (group <= 4) {
        MergeState<4> st;
        st.clear();
        warp_merge_parts<4, 4, false>(st, first, expected, w, n_warps, group, lane);
        warp_merge_stash<4>(st, group, lane, dst);
    } else if (group <= 6) {
        MergeState<6> st;
        st.clear();
        warp_merge_parts<6, 4, false>(st, first, expected, w, n_warps, group, lane);
        warp_merge_stash<6>(st, group, lane, dst);
    } else {
        MergeState<8> st;
        st.clear();
        warp_merge_parts<8, 2, false>(st, first, expected, w, n_warps, group, lane);
        warp_merge_stash<8>(st, group, lane, dst);
    }
}

template <bool kBf16>
__device__ __forceinline__ void warp_merge_finish(const float *stash, int n_warps, int group, int lane, void *out, float *part,
                                                  long long out_row0) {
    if (group <= 4) {
        MergeState<4> st;
        st.clear();
        warp_merge_parts<4, 4, false>(st, stash, n_warps, 0, 1, group, lane);
        warp_merge_store<kBf16, 4>(st, group, lane, out, part, out_row0);
    } else if (group <= 6) {
        MergeState<6> st;
        st.clear();
        warp_merge_parts<6, 4, false>(st, stash, n_warps, 0, 1, group, lane);
        warp_merge_store<kBf16, 6>(st, group, lane, out, part, out_row0);
    } else {
        MergeState<8> st;
        st.clear();
        warp_merge_parts<8, 2, false>(st, stash, n_warps, 0, 1, group, lane);
        warp_merge_store<kBf16, 8>(st, group, lane, out, part, out_row0);
    }
}

} // namespace llaisys::kernels
