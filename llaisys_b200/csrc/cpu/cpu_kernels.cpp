#include "cpu_kernels.hpp"

#include "../common/check.hpp"
#include "../common/dtypes.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <type_traits>
#include <vector>

namespace llaisys::cpu {

using kernels::AttnBatch;
using kernels::AttnOut;
using kernels::KVView;

namespace {

constexpr int kErrBadPage = 1, kErrBadPosition = 2;

template <typename T>
inline float load_f32(const T *p) {
    return utils::cast<float>(*p);
}

template <typename T>
void add_typed(T *c, const T *a, const T *b, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        c[i] = utils::cast<T>(load_f32(a + i) + load_f32(b + i));
    }
}

// (table row, position) -> byte offset of the token's row for kv-head 0, or -1 with the reason in *err.
int64_t slot_offset_bytes(const KVView &kv, size_t elem_size, int32_t seq_row, int32_t pos, int32_t max_blocks,
                          int *err) {
    const int32_t blk = pos / kv.page_size;
    if (pos < 0 || seq_row < 0 || blk >= max_blocks) {
        *err |= kErrBadPosition;
        return -1;
    }
    const int32_t page = kv.block_table ? kv.block_table[int64_t(seq_row) * kv.table_stride + blk] : blk;
    if (page < 0 || page >= kv.num_pages) {
        *err |= kErrBadPage;
        return -1;
    }
    return (int64_t(page) * kv.page_stride + int64_t(pos - blk * kv.page_size) * kv.token_stride) * int64_t(elem_size);
}

template <typename T>
void attention_typed(const KVView &kv, const AttnBatch &b, const T *q, float scale, T *out, float *part, int *err_out) {
    const int d = kv.d, group = b.nh / kv.nkvh;
    // per-row sequence lookup
    const size_t n_rows_q = size_t(b.total_q);
    std::vector<int32_t> row_seq(n_rows_q), row_t(n_rows_q), row_qlen(n_rows_q);
    for (int s = 0, row = 0; s < b.n_seqs; ++s) {
        const int q_len = b.q_starts ? b.q_starts[s + 1] - b.q_starts[s] : b.const_q_len;
        for (int t = 0; t < q_len && row < b.total_q; ++t, ++row) {
            row_seq[row] = s;
            row_t[row] = t;
            row_qlen[row] = q_len;
        }
    }
    int err = 0;
    const int64_t n_items = int64_t(b.total_q) * b.nh;
#pragma omp parallel for schedule(dynamic, 4) reduction(| : err)
    for (int64_t item = 0; item < n_items; ++item) {
        const int row = int(item / b.nh), h = int(item % b.nh);
        const int s = row_seq[row];
        const int kv_len = b.kv_lens ? b.kv_lens[s] : b.const_kv_len;
        const int visible = std::clamp(kv_len - row_qlen[row] + row_t[row] + 1, 0, kv_len);
        const int seq_row = b.seq_ids ? b.seq_ids[s] : s;
        const int kvh = h / group;
        const T *q_row = q + (int64_t(row) * b.nh + h) * d;
        const size_t n_vis = size_t(visible);
        std::vector<float> qf(d), acc(d, 0.f), scores(n_vis);
        std::vector<int64_t> offs(n_vis);
        for (int i = 0; i < d; ++i) {
            qf[i] = load_f32(q_row + i) * scale;
        }
        const T *k_base = static_cast<const T *>(kv.k_base) + int64_t(kvh) * kv.head_stride;
        const T *v_base = static_cast<const T *>(kv.v_base) + int64_t(kvh) * kv.head_stride;
        float m = -std::numeric_limits<float>::infinity();
        for (int j = 0; j < visible; ++j) {
            const int64_t off_b = slot_offset_bytes(kv, sizeof(T), seq_row, j, std::numeric_limits<int32_t>::max(), &err);
            offs[j] = off_b < 0 ? -1 : off_b / int64_t(sizeof(T));
            if (off_b < 0) {
                scores[j] = -std::numeric_limits<float>::infinity();
                continue;
            }
            const T *k_row = k_base + offs[j];
            float dot = 0.f;
            for (int i = 0; i < d; ++i) {
                dot += qf[i] * load_f32(k_row + i);
            }
            scores[j] = dot;
            m = std::max(m, dot);
        }
        float l = 0.f;
        for (int j = 0; j < visible; ++j) {
            if (offs[j] < 0) {
                continue;
            }
            const float p = std::exp(scores[j] - m);
            l += p;
            const T *v_row = v_base + offs[j];
            for (int i = 0; i < d; ++i) {
                acc[i] += p * load_f32(v_row + i);
            }
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int64_t o_row = int64_t(row) * b.nh + h;
        if (part != nullptr) {
            float *dst = part + o_row * (d + 2);
            for (int i = 0; i < d; ++i) {
                dst[i] = acc[i] * inv;
            }
            dst[d] = m;
            dst[d + 1] = l;
        } else {
            T *dst = out + o_row * d;
            for (int i = 0; i < d; ++i) {
                dst[i] = utils::cast<T>(acc[i] * inv);
            }
        }
    }
    *err_out = err;
}

template <typename T>
void lse_merge_typed(T *out, const float *parts, int n_parts, int n_rows, int d) {
    const int64_t row_stride = d + 2, part_stride = int64_t(n_rows) * row_stride;
    for (int r = 0; r < n_rows; ++r) {
        const float *base = parts + int64_t(r) * row_stride;
        float m_all = -std::numeric_limits<float>::infinity();
        for (int p = 0; p < n_parts; ++p) {
            if (base[p * part_stride + d + 1] > 0.f) {
                m_all = std::max(m_all, base[p * part_stride + d]);
            }
        }
        const size_t np = size_t(n_parts);
        std::vector<float> w(np, 0.f);
        float l_all = 0.f;
        for (int p = 0; p < n_parts; ++p) {
            const float l = base[p * part_stride + d + 1];
            if (l > 0.f) {
                w[p] = l * std::exp(base[p * part_stride + d] - m_all);
                l_all += w[p];
            }
        }
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        for (int i = 0; i < d; ++i) {
            float o = 0.f;
            for (int p = 0; p < n_parts; ++p) {
                if (w[p] != 0.f) {
                    o += w[p] * base[p * part_stride + i];
                }
            }
            out[int64_t(r) * d + i] = utils::cast<T>(o * inv);
        }
    }
}

} // namespace

void add(llaisysDataType_t dtype, void *c, const void *a, const void *b, size_t n) {
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        return add_typed(static_cast<float *>(c), static_cast<const float *>(a), static_cast<const float *>(b), n);
    case LLAISYS_DTYPE_F16:
        return add_typed(static_cast<fp16_t *>(c), static_cast<const fp16_t *>(a), static_cast<const fp16_t *>(b), n);
    case LLAISYS_DTYPE_BF16:
        return add_typed(static_cast<bf16_t *>(c), static_cast<const bf16_t *>(a), static_cast<const bf16_t *>(b), n);
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
}

void rearrange(size_t elem_size, size_t ndim, const size_t *shape, const ptrdiff_t *dst_strides,
               const ptrdiff_t *src_strides, void *dst, const void *src) {
    size_t total = 1;
    for (size_t i = 0; i < ndim; ++i) {
        total *= shape[i];
    }
    if (total == 0) {
        return;
    }
    std::vector<size_t> idx(ndim, 0);
    auto *d = static_cast<std::byte *>(dst);
    const auto *s = static_cast<const std::byte *>(src);
    ptrdiff_t d_off = 0, s_off = 0;
    for (size_t n = 0; n < total; ++n) {
        std::memcpy(d + d_off * ptrdiff_t(elem_size), s + s_off * ptrdiff_t(elem_size), elem_size);
        // odometer increment, keeping both offsets in step
        for (size_t k = ndim; k-- > 0;) {
            ++idx[k];
            d_off += dst_strides[k];
            s_off += src_strides[k];
            if (idx[k] < shape[k]) {
                break;
            }
            d_off -= dst_strides[k] * ptrdiff_t(shape[k]);
            s_off -= src_strides[k] * ptrdiff_t(shape[k]);
            idx[k] = 0;
        }
    }
}

int paged_append(size_t elem_size, const KVView &kv, const void *k_rows, const void *v_rows, const int32_t *seq_ids,
                 const int32_t *positions, int32_t n_rows, int32_t max_blocks) {
    int err = 0;
    const size_t head_row = size_t(kv.d) * elem_size;
    const auto *ks = static_cast<const std::byte *>(k_rows);
    const auto *vs = static_cast<const std::byte *>(v_rows);
    auto *kp = static_cast<std::byte *>(kv.k_base);
    auto *vp = static_cast<std::byte *>(kv.v_base);
    for (int32_t r = 0; r < n_rows; ++r) {
        const int64_t off = slot_offset_bytes(kv, elem_size, seq_ids[r], positions[r], max_blocks, &err);
        if (off < 0) {
            continue;
        }
        for (int32_t h = 0; h < kv.nkvh; ++h) {
            const int64_t dst = off + int64_t(h) * kv.head_stride * int64_t(elem_size);
            const size_t src = (size_t(r) * kv.nkvh + h) * head_row;
            std::memcpy(kp + dst, ks + src, head_row);
            std::memcpy(vp + dst, vs + src, head_row);
        }
    }
    return err;
}

int paged_gather(size_t elem_size, const KVView &kv, int32_t seq_row, int32_t n_tokens, void *k_out, void *v_out) {
    int err = 0;
    const size_t head_row = size_t(kv.d) * elem_size;
    auto *ko = static_cast<std::byte *>(k_out);
    auto *vo = static_cast<std::byte *>(v_out);
    const auto *kp = static_cast<const std::byte *>(kv.k_base);
    const auto *vp = static_cast<const std::byte *>(kv.v_base);
    const int32_t max_blocks = kv.block_table ? kv.table_stride : std::numeric_limits<int32_t>::max();
    for (int32_t t = 0; t < n_tokens; ++t) {
        const int64_t off = slot_offset_bytes(kv, elem_size, seq_row, t, max_blocks, &err);
        if (off < 0) {
            continue;
        }
        for (int32_t h = 0; h < kv.nkvh; ++h) {
            const int64_t src = off + int64_t(h) * kv.head_stride * int64_t(elem_size);
            const size_t dst = (size_t(t) * kv.nkvh + h) * head_row;
            std::memcpy(ko + dst, kp + src, head_row);
            std::memcpy(vo + dst, vp + src, head_row);
        }
    }
    return err;
}

int attention(llaisysDataType_t dtype, const KVView &kv, const AttnBatch &batch, const void *q, float scale,
              const AttnOut &out) {
    if (batch.total_q <= 0 || batch.nh <= 0) {
        return 0;
    }
    CHECK_ARGUMENT(kv.nkvh > 0 && batch.nh % kv.nkvh == 0, "attention: nh must be a multiple of nkvh");
    int err = 0;
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        attention_typed(kv, batch, static_cast<const float *>(q), scale, static_cast<float *>(out.out), out.part, &err);
        break;
    case LLAISYS_DTYPE_F16:
        attention_typed(kv, batch, static_cast<const fp16_t *>(q), scale, static_cast<fp16_t *>(out.out), out.part, &err);
        break;
    case LLAISYS_DTYPE_BF16:
        attention_typed(kv, batch, static_cast<const bf16_t *>(q), scale, static_cast<bf16_t *>(out.out), out.part, &err);
        break;
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
    return err;
}

void lse_merge(llaisysDataType_t dtype, void *out, const float *parts, int32_t n_parts, int32_t n_rows, int32_t d) {
    switch (dtype) {
    case LLAISYS_DTYPE_F32:
        return lse_merge_typed(static_cast<float *>(out), parts, n_parts, n_rows, d);
    case LLAISYS_DTYPE_F16:
        return lse_merge_typed(static_cast<fp16_t *>(out), parts, n_parts, n_rows, d);
    case LLAISYS_DTYPE_BF16:
        return lse_merge_typed(static_cast<bf16_t *>(out), parts, n_parts, n_rows, d);
    default:
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);
    }
}


// ---- the remaining operators -----------------------------------------------------------------------------------

namespace {

template <typename T>
void argmax_typed(int64_t *idx_out, T *val_out, const T *vals, size_t rows, size_t n) {
#pragma omp parallel for if (rows > 1)
    for (int64_t r = 0; r < int64_t(rows); ++r) {
        const T *row = vals + size_t(r) * n;
        size_t best = 0;
        float best_v = load_f32(row);
        for (size_t i = 1; i < n; ++i) {
            const float v = load_f32(row + i);
            if (v > best_v) { // strict: the first of equal maxima wins
                best_v = v;
                best = i;
            }
        }
        idx_out[r] = int64_t(best);
        if (val_out != nullptr) {
            val_out[r] = row[best];
        }
    }
}

template <typename T>
void linear_typed(T *out, const T *in, const T *w, const T *bias, size_t m, size_t n, size_t k, bool accumulate) {
    // Convert once to f32 rows (bf16/f16 conversions are the expensive part on the host), then blocked dot products
    // with a double accumulator so that the reference's f32 tolerance (1e-5 relative at K = 4096) holds.
    std::vector<float> in_f(m * k), w_f;
    for (size_t i = 0; i < m * k; ++i) {
        in_f[i] = load_f32(in + i);
    }
    const bool convert_w = !std::is_same_v<T, float>;
    if (convert_w) {
        w_f.resize(n * k);
#pragma omp parallel for
        for (int64_t i = 0; i < int64_t(n * k); ++i) {
            w_f[size_t(i)] = load_f32(w + i);
        }
    }
    const float *wp = convert_w ? w_f.data() : reinterpret_cast<const float *>(w);
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < int64_t(m); ++i) {
        for (int64_t j = 0; j < int64_t(n); ++j) {
            const float *a = in_f.data() + size_t(i) * k;
            const float *b = wp + size_t(j) * k;
            double acc = 0.0;
            size_t x = 0;
            for (; x + 8 <= k; x += 8) {
                float part = 0.f;
                for (size_t u = 0; u < 8; ++u) {
                    part += a[x + u] * b[x + u];
                }
                acc += part;
            }
            for (; x < k; ++x) {
                acc += double(a[x]) * b[x];
            }
            if (bias != nullptr) {
                acc += load_f32(bias + j);
            }
            if (accumulate) {
                acc += load_f32(out + size_t(i) * n + size_t(j));
            }
            out[size_t(i) * n + size_t(j)] = utils::cast<T>(float(acc));
        }
    }
}

template <typename T>
void rms_norm_typed(T *out, const T *in, const T *w, float eps, size_t rows, size_t d) {
#pragma omp parallel for if (rows > 8)
    for (int64_t r = 0; r < int64_t(rows); ++r) {
        const T *x = in + size_t(r) * d;
        double ss = 0.0;
        for (size_t i = 0; i < d; ++i) {
            const float v = load_f32(x + i);
            ss += double(v) * v;
        }
        const float inv = 1.f / std::sqrt(float(ss / double(d)) + eps);
        for (size_t i = 0; i < d; ++i) {
            out[size_t(r) * d + i] = utils::cast<T>(load_f32(w + i) * load_f32(x + i) * inv);
        }
    }
}

template <typename T>
void rope_typed(T *out, const T *in, const int64_t *pos, float theta, size_t seq, size_t heads, size_t d) {
    const size_t half = d / 2;
    std::vector<float> divisor(half);
    for (size_t j = 0; j < half; ++j) {
        divisor[j] = std::pow(theta, 2.f * float(j) / float(d)); // the divisor theta^(2j/d), in f32 like the oracle
    }
#pragma omp parallel for if (seq * heads > 64)
    for (int64_t s = 0; s < int64_t(seq); ++s) {
        const float p = float(pos[s]);
        for (size_t h = 0; h < heads; ++h) {
            const T *x = in + (size_t(s) * heads + h) * d;
            T *y = out + (size_t(s) * heads + h) * d;
            for (size_t j = 0; j < half; ++j) {
                const float ang = p / divisor[j];
                const float sn = std::sin(ang), cs = std::cos(ang);
                const float a = load_f32(x + j), b = load_f32(x + j + half);
                y[j] = utils::cast<T>(a * cs - b * sn);
                y[j + half] = utils::cast<T>(b * cs + a * sn);
            }
        }
    }
}

template <typename T>
void swiglu_packed_typed(T *out, const T *gu, size_t rows, size_t di) {
#pragma omp parallel for if (rows * di > 65536)
    for (int64_t r = 0; r < int64_t(rows); ++r) {
        for (size_t i = 0; i < di; ++i) {
            const float g = load_f32(gu + size_t(r) * 2 * di + i), u = load_f32(gu + size_t(r) * 2 * di + di + i);
            out[size_t(r) * di + i] = utils::cast<T>(u * (g / (1.f + std::exp(-g))));
        }
    }
}

// The fused step before attention (same arithmetic as the CUDA kernel): bias, rotary embedding of the q and k heads,
// q to its own tensor, k and v into their page slots. f32 arithmetic, one rounding.
template <typename T>
int paged_rope_append_typed(const KVView &kv, T *q_out, const T *qkv, const T *bias, const int32_t *seq_ids,
                            const int32_t *positions, int32_t n_rows, int32_t nh, float theta, int32_t max_blocks) {
    int err = 0;
    const int32_t d = kv.d, half = d / 2, heads = nh + 2 * kv.nkvh;
    std::vector<float> divisor(static_cast<size_t>(half));
    for (int32_t j = 0; j < half; ++j) {
        divisor[size_t(j)] = std::pow(theta, 2.f * float(j) / float(d));
    }
    auto *kp = static_cast<std::byte *>(kv.k_base);
    auto *vp = static_cast<std::byte *>(kv.v_base);
    for (int32_t r = 0; r < n_rows; ++r) {
        const int64_t off = slot_offset_bytes(kv, sizeof(T), seq_ids[r], positions[r], max_blocks, &err);
        const float p = float(positions[r]);
        for (int32_t h = 0; h < heads; ++h) {
            const T *x = qkv + (size_t(r) * heads + h) * d;
            const T *b = bias ? bias + size_t(h) * d : nullptr;
            const bool is_q = h < nh, is_v = h >= nh + kv.nkvh;
            T *y = nullptr;
            if (is_q) {
                y = q_out + (size_t(r) * nh + h) * d;
            } else if (off >= 0) {
                const int32_t kvh = is_v ? h - nh - kv.nkvh : h - nh;
                y = reinterpret_cast<T *>((is_v ? vp : kp) + off + int64_t(kvh) * kv.head_stride * int64_t(sizeof(T)));
            } else {
                continue;
            }
            for (int32_t j = 0; j < half; ++j) {
                float lo = load_f32(x + j), hi = load_f32(x + j + half);
                if (b != nullptr) {
                    lo += load_f32(b + j);
                    hi += load_f32(b + j + half);
                }
                if (!is_v) {
                    const float ang = p / divisor[size_t(j)];
                    const float sn = std::sin(ang), cs = std::cos(ang);
                    const float a0 = lo, b0 = hi;
                    lo = a0 * cs - b0 * sn;
                    hi = b0 * cs + a0 * sn;
                }
                y[j] = utils::cast<T>(lo);
                y[j + half] = utils::cast<T>(hi);
            }
        }
    }
    return err;
}

template <typename T>
void swiglu_typed(T *out, const T *gate, const T *up, size_t n) {
#pragma omp parallel for if (n > 65536)
    for (int64_t i = 0; i < int64_t(n); ++i) {
        const float g = load_f32(gate + i);
        out[i] = utils::cast<T>(load_f32(up + i) * (g / (1.f + std::exp(-g))));
    }
}

} // namespace

#define LLAISYS_DISPATCH_FLOAT(dtype, CALL)            \
    switch (dtype) {                                   \
    case LLAISYS_DTYPE_F32: {                          \
        using T = float;                               \
        CALL;                                          \
        break;                                         \
    }                                                  \
    case LLAISYS_DTYPE_F16: {                          \
        using T = fp16_t;                              \
        CALL;                                          \
        break;                                         \
    }                                                  \
    case LLAISYS_DTYPE_BF16: {                         \
        using T = bf16_t;                              \
        CALL;                                          \
        break;                                         \
    }                                                  \
    default:                                           \
        EXCEPTION_UNSUPPORTED_DATATYPE(dtype);         \
    }

void argmax_rows(llaisysDataType_t dtype, int64_t *idx_out, void *val_out, const void *vals, size_t rows, size_t n) {
    LLAISYS_DISPATCH_FLOAT(dtype, argmax_typed(idx_out, static_cast<T *>(val_out), static_cast<const T *>(vals), rows, n));
}

void embedding(size_t elem_size, void *out, const int64_t *index, const void *weight, size_t n, size_t d, size_t vocab) {
    const size_t row = d * elem_size;
    for (size_t i = 0; i < n; ++i) {
        CHECK_ARGUMENT(index[i] >= 0 && size_t(index[i]) < vocab, "embedding: index out of range");
        std::memcpy(static_cast<std::byte *>(out) + i * row, static_cast<const std::byte *>(weight) + size_t(index[i]) * row, row);
    }
}

void linear(llaisysDataType_t dtype, void *out, const void *in, const void *weight, const void *bias, size_t m, size_t n,
            size_t k, bool accumulate) {
    LLAISYS_DISPATCH_FLOAT(dtype, linear_typed(static_cast<T *>(out), static_cast<const T *>(in), static_cast<const T *>(weight),
                                               static_cast<const T *>(bias), m, n, k, accumulate));
}

void swiglu_packed(llaisysDataType_t dtype, void *out, const void *gate_up, size_t rows, size_t di) {
    LLAISYS_DISPATCH_FLOAT(dtype, swiglu_packed_typed(static_cast<T *>(out), static_cast<const T *>(gate_up), rows, di));
}

int paged_rope_append(llaisysDataType_t dtype, const kernels::KVView &kv, void *q_out, const void *qkv, const void *bias,
                      const int32_t *seq_ids, const int32_t *positions, int32_t n_rows, int32_t nh, float theta,
                      int32_t max_blocks) {
    LLAISYS_DISPATCH_FLOAT(dtype, return paged_rope_append_typed(kv, static_cast<T *>(q_out), static_cast<const T *>(qkv),
                                                                 static_cast<const T *>(bias), seq_ids, positions, n_rows, nh,
                                                                 theta, max_blocks));
    return 0;
}

void rms_norm(llaisysDataType_t dtype, void *out, const void *in, const void *weight, float eps, size_t rows, size_t d) {
    LLAISYS_DISPATCH_FLOAT(dtype, rms_norm_typed(static_cast<T *>(out), static_cast<const T *>(in),
                                                 static_cast<const T *>(weight), eps, rows, d));
}

void rope(llaisysDataType_t dtype, void *out, const void *in, const int64_t *pos, float theta, size_t seq, size_t heads,
          size_t d) {
    LLAISYS_DISPATCH_FLOAT(dtype, rope_typed(static_cast<T *>(out), static_cast<const T *>(in), pos, theta, seq, heads, d));
}

void swiglu(llaisysDataType_t dtype, void *out, const void *gate, const void *up, size_t n) {
    LLAISYS_DISPATCH_FLOAT(dtype, swiglu_typed(static_cast<T *>(out), static_cast<const T *>(gate), static_cast<const T *>(up), n));
}

} // namespace llaisys::cpu
