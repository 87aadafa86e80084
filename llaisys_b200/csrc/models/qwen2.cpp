#include "qwen2.hpp"

#include "../common/check.hpp"
#include "../common/dtypes.hpp"
#include "../cpu/cpu_kernels.hpp"
#include "llaisys/paged_kv.h"
#ifdef ENABLE_NVIDIA_API
#include "../kernels/kernels.hpp"
#endif

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>

namespace llaisys::models {

namespace {
constexpr size_t kPageSize = 16;
constexpr size_t kNotLive = std::numeric_limits<size_t>::max();

[[noreturn]] void fail(int code, const std::string &msg) { throw kv::StatusError(code, msg); }
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
} // namespace

// ---- construction -------------------------------------------------------------------------------------------------

namespace {
LlaisysQwen2Meta shard_meta(LlaisysQwen2Meta meta, int tp_rank, int tp_world) {
    if (tp_world < 1 || tp_rank < 0 || tp_rank >= tp_world) {
        fail(LLAISYS_E_INVALID, "qwen2: bad tensor-parallel rank or world size");
    }
    const size_t w = size_t(tp_world);
    if (meta.nkvh % w != 0 || meta.nh % w != 0 || meta.di % w != 0) {
        fail(LLAISYS_E_INVALID, "qwen2: the tensor-parallel world size must divide nkvh, nh and di");
    }
    meta.nh /= w;
    meta.nkvh /= w;
    meta.di /= w;
    return meta;
}
} // namespace

Qwen2::Qwen2(const LlaisysQwen2Meta &global_meta, llaisysDeviceType_t device, int device_id, int tp_rank, int tp_world)
    : _meta(shard_meta(global_meta, tp_rank, tp_world)), _tp_rank(tp_rank), _tp_world(tp_world), _device(device),
      _device_id(device_id) {
    const LlaisysQwen2Meta &meta = _meta;
    if (meta.dtype != LLAISYS_DTYPE_F32 && meta.dtype != LLAISYS_DTYPE_F16 && meta.dtype != LLAISYS_DTYPE_BF16) {
        fail(LLAISYS_E_INVALID, "qwen2: dtype must be F32, F16 or BF16");
    }
    if (meta.nlayer == 0 || meta.hs == 0 || meta.nh == 0 || meta.nkvh == 0 || meta.dh == 0 || meta.di == 0 || meta.voc == 0 ||
        meta.nh % meta.nkvh != 0 || meta.dh % 2 != 0) {
        fail(LLAISYS_E_INVALID, "qwen2: inconsistent model dimensions");
    }
    _elem = utils::dsize(meta.dtype);
    _on_gpu = device != LLAISYS_DEVICE_CPU;
    auto &rt = enter();
    _stream = rt.stream();

    const size_t L = meta.nlayer, hs = meta.hs, qd = meta.nh * meta.dh, kd = meta.nkvh * meta.dh, di = meta.di;
    _weights.in_embed = makeWeight({meta.voc, hs});
    _weights.out_embed = makeWeight({meta.voc, hs});
    _weights.out_norm_w = makeWeight({hs});
    for (auto &v : _per_layer) {
        v.resize(L);
    }
    _qkv_w.resize(L);
    _qkv_b.resize(L);
    _gate_up_w.resize(L);
    const std::vector<std::byte> zeros((qd + 2 * kd) * _elem);
    for (size_t l = 0; l < L; ++l) {
        _qkv_w[l] = Tensor::create({qd + 2 * kd, hs}, meta.dtype, device, device_id);
        _qkv_b[l] = Tensor::create({qd + 2 * kd}, meta.dtype, device, device_id);
        _qkv_b[l]->load(zeros.data()); // a caller that loads no biases gets none
        _gate_up_w[l] = Tensor::create({2 * di, hs}, meta.dtype, device, device_id);
        _per_layer[0][l] = makeWeight({hs});
        _per_layer[1][l] = wrap(_qkv_w[l]->slice(0, 0, qd));
        _per_layer[2][l] = wrap(_qkv_b[l]->slice(0, 0, qd));
        _per_layer[3][l] = wrap(_qkv_w[l]->slice(0, qd, qd + kd));
        _per_layer[4][l] = wrap(_qkv_b[l]->slice(0, qd, qd + kd));
        _per_layer[5][l] = wrap(_qkv_w[l]->slice(0, qd + kd, qd + 2 * kd));
        _per_layer[6][l] = wrap(_qkv_b[l]->slice(0, qd + kd, qd + 2 * kd));
        _per_layer[7][l] = makeWeight({hs, qd});
        _per_layer[8][l] = makeWeight({hs});
        _per_layer[9][l] = wrap(_gate_up_w[l]->slice(0, 0, di));
        _per_layer[10][l] = wrap(_gate_up_w[l]->slice(0, di, 2 * di));
        _per_layer[11][l] = makeWeight({hs, di});
    }
    _weights.attn_norm_w = _per_layer[0].data();
    _weights.attn_q_w = _per_layer[1].data();
    _weights.attn_q_b = _per_layer[2].data();
    _weights.attn_k_w = _per_layer[3].data();
    _weights.attn_k_b = _per_layer[4].data();
    _weights.attn_v_w = _per_layer[5].data();
    _weights.attn_v_b = _per_layer[6].data();
    _weights.attn_o_w = _per_layer[7].data();
    _weights.mlp_norm_w = _per_layer[8].data();
    _weights.mlp_gate_w = _per_layer[9].data();
    _weights.mlp_up_w = _per_layer[10].data();
    _weights.mlp_down_w = _per_layer[11].data();
}

void Qwen2::dropStepGraphs() {
#ifdef ENABLE_NVIDIA_API
    for (StepGraph &g : _step_graphs) {
        if (g.exec != nullptr) {
            kernels::graph_destroy(g.exec);
        }
    }
#endif
    _step_graphs.clear();
}

Qwen2::~Qwen2() {
    dropStepGraphs();
    for (ModelObserver *o : std::vector<ModelObserver *>(_observers)) {
        o->modelDestroyed();
    }
    for (llaisysTensor_t h : _all_weights) {
        delete h;
    }
}

core::Runtime &Qwen2::enter() const {
    auto &ctx = core::context();
    ctx.setDevice(_device, _device_id);
    return ctx.runtime();
}

llaisysTensor_t Qwen2::wrap(tensor_t t) {
    auto *h = new LlaisysTensor{std::move(t)};
    _all_weights.push_back(h);
    return h;
}

llaisysTensor_t Qwen2::makeWeight(const std::vector<size_t> &shape) {
    return wrap(Tensor::create(shape, _meta.dtype, _device, _device_id));
}

std::vector<Qwen2::Layer> Qwen2::layerPointers() const {
    std::vector<Layer> layers(_meta.nlayer);
    for (size_t l = 0; l < _meta.nlayer; ++l) {
        auto p = [&](int w) { return static_cast<const std::byte *>(_per_layer[w][l]->tensor->data()); };
        auto packed = [](const tensor_t &t) { return static_cast<const std::byte *>(t->data()); };
        layers[l] = Layer{p(0), packed(_qkv_w[l]), packed(_qkv_b[l]), p(7), p(8), packed(_gate_up_w[l]), p(11)};
    }
    return layers;
}

// ---- cache and sequences --------------------------------------------------------------------------------------------

void Qwen2::configureCache(size_t max_seqs, size_t max_tokens) {
    if (max_seqs == 0 || max_tokens == 0) {
        fail(LLAISYS_E_INVALID, "qwen2: cache sizes must be positive");
    }
    kv::PagedKVConfig cfg;
    cfg.device_type = _device;
    cfg.device_id = _device_id;
    cfg.dtype = _meta.dtype;
    cfg.nlayer = _meta.nlayer;
    cfg.page_size = kPageSize;
    cfg.nkvh = _meta.nkvh;
    cfg.head_dim = _meta.dh;
    cfg.max_seqs = max_seqs;
    cfg.max_pages_per_seq = (max_tokens + kPageSize - 1) / kPageSize;
    cfg.num_pages = cfg.max_seqs * cfg.max_pages_per_seq;
    dropStepGraphs();
    _cache = std::make_unique<kv::PagedKV>(cfg);
    // [bias + rope + append] -> decode attention run as a programmatic pair: the attention kernel's set-up and its copies
    // of older pages overlap the append (which writes each sequence's last page only, as the overlap contract asks)
    _cache->setLaunchOverlap(_on_gpu);
    _max_tokens_per_seq = cfg.max_pages_per_seq * kPageSize;
    _seq_len.assign(max_seqs, kNotLive);
    _seq_tokens.assign(max_seqs, {});
    _implicit_seq = -1;
}

size_t &Qwen2::seqLen(int32_t seq) {
    if (!_cache || seq < 0 || size_t(seq) >= _seq_len.size() || _seq_len[seq] == kNotLive) {
        fail(LLAISYS_E_NO_SEQ, "qwen2: sequence " + std::to_string(seq) + " does not exist");
    }
    return _seq_len[seq];
}

int32_t Qwen2::seqAdd() {
    if (!_cache) {
        fail(LLAISYS_E_INVALID, "qwen2: call llaisysQwen2ModelConfigureCache first");
    }
    const int32_t s = _cache->seqAdd();
    _seq_len[s] = 0;
    _seq_tokens[s].clear();
    return s;
}

int32_t Qwen2::seqAddWithPrefix(const int64_t *tokens, size_t n, size_t *matched) {
    const int32_t s = seqAdd();
    size_t got = 0;
    if (n > 1 && tokens != nullptr) {
        try {
            got = _cache->seqMatchPrefix(s, tokens, n - 1); // whole pages inside the first n - 1 tokens
        } catch (...) {
            seqFree(s);
            throw;
        }
        _seq_tokens[s].assign(tokens, tokens + got);
    }
    _seq_len[s] = got;
    if (matched != nullptr) {
        *matched = got;
    }
    return s;
}

void Qwen2::seqReserve(int32_t seq, size_t n_tokens) {
    seqLen(seq);
    if (n_tokens > _max_tokens_per_seq) {
        fail(LLAISYS_E_INVALID, "qwen2: sequence would exceed the configured maximum length");
    }
    _cache->seqReserve(seq, n_tokens);
}

// The sequence now holds K/V for n more tokens: remember their ids and publish the pages they completed.
void Qwen2::recordTokens(int32_t seq, const int64_t *tokens, size_t n) {
    std::vector<int64_t> &held = _seq_tokens[seq];
    const size_t before = held.size() / kPageSize;
    held.insert(held.end(), tokens, tokens + n);
    if (held.size() / kPageSize != before) {
        _cache->seqPublish(seq, held.data(), held.size());
    }
}

void Qwen2::seqFree(int32_t seq) {
    seqLen(seq);
    _cache->seqFree(seq);
    _seq_len[seq] = kNotLive;
    _seq_tokens[seq].clear();
    if (seq == _implicit_seq) {
        _implicit_seq = -1;
    }
}

void Qwen2::reset() {
    if (_implicit_seq >= 0) {
        seqFree(_implicit_seq);
    }
}

int64_t Qwen2::infer(const int64_t *tokens, size_t n) {
    if (n == 0 || tokens == nullptr) {
        fail(LLAISYS_E_INVALID, "qwen2: infer needs at least one token");
    }
    if (!_cache) {
        configureCache(1, std::max<size_t>(_meta.maxseq, n + 1));
    }
    if (_implicit_seq < 0) {
        _implicit_seq = seqAdd();
    }
    const int32_t n32 = int32_t(n);
    int64_t next = 0;
    step(&_implicit_seq, &n32, 1, tokens, &next);
    return next;
}

// ---- workspace -------------------------------------------------------------------------------------------------------

void Qwen2::ensureWorkspace(size_t n_tokens, size_t n_seqs) {
    auto &rt = enter();
    if (n_tokens > _ws_tokens) {
        ++_generation;
        _ws_tokens = n_tokens;
        const size_t hs = _meta.hs, qd = _meta.nh * _meta.dh, kd = _meta.nkvh * _meta.dh;
        _x = rt.allocateDeviceStorage(n_tokens * hs * _elem);
        _h = rt.allocateDeviceStorage(n_tokens * hs * _elem);
        _qkv = rt.allocateDeviceStorage(n_tokens * (qd + 2 * kd) * _elem);
        _q = rt.allocateDeviceStorage(n_tokens * qd * _elem);
        _attn = rt.allocateDeviceStorage(n_tokens * qd * _elem);
        _gate_up = rt.allocateDeviceStorage(n_tokens * 2 * _meta.di * _elem);
        _act = rt.allocateDeviceStorage(n_tokens * _meta.di * _elem);
    }
    if (n_seqs > _ws_seqs) {
        ++_generation;
        _ws_seqs = n_seqs;
        _x_last = rt.allocateDeviceStorage(n_seqs * _meta.hs * _elem);
        _logits = rt.allocateDeviceStorage(n_seqs * _meta.voc * _elem);
        // keys and counters of the split argmax: zero once, the kernel leaves them zero
        _argmax_scratch = rt.allocateDeviceStorage(n_seqs * 12);
        const std::vector<std::byte> zeros(n_seqs * 12);
        copyToDevice(_argmax_scratch->memory(), zeros.data(), zeros.size());
    }
    // tokens, pos64, last_rows, next (int64) then seq32, pos32, kv_lens, q_starts, seq_list (int32), 16-byte aligned
    const size_t need = align_up(n_tokens * 8, 16) * 2 + align_up(n_seqs * 8, 16) * 2 + align_up(n_tokens * 4, 16) * 2 +
                        align_up(n_seqs * 4, 16) * 2 + align_up((n_seqs + 1) * 4, 16);
    if (need > _meta_bytes) {
        ++_generation;
        _meta_bytes = need * 2;
        _meta_block = rt.allocateDeviceStorage(_meta_bytes);
    }
}

Qwen2::StepArrays Qwen2::carveStepArrays(size_t n_tokens, size_t n_seqs) {
    StepArrays a;
    size_t at = 0;
    auto take = [&](size_t bytes) {
        const size_t here = at;
        at += align_up(bytes, 16);
        return here;
    };
    std::byte *base = _meta_block->memory();
    a.tokens = reinterpret_cast<int64_t *>(base + take(n_tokens * 8));
    a.pos64 = reinterpret_cast<int64_t *>(base + take(n_tokens * 8));
    a.last_rows = reinterpret_cast<int64_t *>(base + take(n_seqs * 8));
    a.next = reinterpret_cast<int64_t *>(base + take(n_seqs * 8));
    a.seq32 = reinterpret_cast<int32_t *>(base + take(n_tokens * 4));
    a.pos32 = reinterpret_cast<int32_t *>(base + take(n_tokens * 4));
    a.kv_lens = reinterpret_cast<int32_t *>(base + take(n_seqs * 4));
    a.seq_list = reinterpret_cast<int32_t *>(base + take(n_seqs * 4));
    a.q_starts = reinterpret_cast<int32_t *>(base + take((n_seqs + 1) * 4));
    return a;
}

void Qwen2::copyToDevice(void *dst, const void *src, size_t bytes) {
    auto &rt = enter();
    if (_on_gpu) {
        rt.api()->memcpy_async(dst, src, bytes, LLAISYS_MEMCPY_H2D, _stream);
    } else {
        std::memcpy(dst, src, bytes);
    }
}

void Qwen2::copyToHost(void *dst, const void *src, size_t bytes) {
    auto &rt = enter();
    if (_on_gpu) {
        rt.api()->memcpy_async(dst, src, bytes, LLAISYS_MEMCPY_D2H, _stream);
        rt.synchronize();
    } else {
        std::memcpy(dst, src, bytes);
    }
}

// ---- operator shims ----------------------------------------------------------------------------------------------------

#ifdef ENABLE_NVIDIA_API
#define QWEN2_DISPATCH(CPU_CALL, CUDA_CALL) \
    if (_on_gpu) {                          \
        CUDA_CALL;                          \
    } else {                                \
        CPU_CALL;                           \
    }
#else
#define QWEN2_DISPATCH(CPU_CALL, CUDA_CALL) CPU_CALL;
#endif

void Qwen2::opEmbedding(void *out, const int64_t *idx, const void *w, size_t n, size_t d, size_t vocab) {
    QWEN2_DISPATCH(cpu::embedding(_elem, out, idx, w, n, d, vocab), kernels::embedding(_stream, _elem, out, idx, w, n, d, vocab));
}
void Qwen2::opLinear(void *out, const void *in, const void *w, size_t m, size_t n, size_t k, bool accumulate) {
    QWEN2_DISPATCH(cpu::linear(_meta.dtype, out, in, w, nullptr, m, n, k, accumulate),
                   kernels::linear(_stream, _meta.dtype, out, in, w, nullptr, m, n, k, accumulate));
}
void Qwen2::opRmsNorm(void *out, const void *in, const void *w, size_t rows, size_t d) {
    QWEN2_DISPATCH(cpu::rms_norm(_meta.dtype, out, in, w, _meta.epsilon, rows, d),
                   kernels::rms_norm(_stream, _meta.dtype, out, in, w, _meta.epsilon, rows, d));
}
void Qwen2::opSwigluPacked(void *out, const void *gate_up, size_t rows, size_t di) {
    QWEN2_DISPATCH(cpu::swiglu_packed(_meta.dtype, out, gate_up, rows, di),
                   kernels::swiglu_packed(_stream, _meta.dtype, out, gate_up, rows, di));
}
void Qwen2::opAdd(void *c, const void *a, const void *b, size_t n) {
    QWEN2_DISPATCH(cpu::add(_meta.dtype, c, a, b, n), kernels::add(_stream, _meta.dtype, c, a, b, n));
}

void Qwen2::setCollective(std::unique_ptr<comm::Collective> c) {
    if (!c || c->rank() != _tp_rank || c->world() != _tp_world) {
        fail(LLAISYS_E_INVALID, "qwen2: the collective's rank / world size differ from the model's");
    }
    _tp = std::move(c);
}

void Qwen2::projectIntoStream(void *x, void *tmp, const void *in, const void *w, size_t m, size_t n, size_t k) {
    if (_tp_world == 1) {
        opLinear(x, in, w, m, n, k, true); // the residual add folded into the projection
        return;
    }
    if (!_tp) {
        fail(LLAISYS_E_INVALID, "qwen2: a sharded model needs its all-reduce (llaisysQwen2ModelSetAllReduce...) before the first step");
    }
    opLinear(tmp, in, w, m, n, k);
    _tp->allReduceSum(tmp, m * n, _meta.dtype, _stream);
    opAdd(x, x, tmp, m * n);
}

void Qwen2::opArgmax(int64_t *idx, const void *vals, size_t rows, size_t n) {
    QWEN2_DISPATCH(cpu::argmax_rows(_meta.dtype, idx, nullptr, vals, rows, n),
                   kernels::argmax_rows_split(_stream, _meta.dtype, idx, vals, rows, n, _argmax_scratch->memory()));
}

// ---- the network ---------------------------------------------------------------------------------------------------------

void Qwen2::forward(const StepArrays &a, size_t T, size_t n_seqs, size_t max_q_len, size_t max_kv_len, bool decode_only) {
    const size_t hs = _meta.hs, qd = _meta.nh * _meta.dh, kd = _meta.nkvh * _meta.dh, di = _meta.di;
    const float scale = 1.f / std::sqrt(float(_meta.dh));
    std::byte *x = _x->memory(), *h = _h->memory(), *qkv = _qkv->memory(), *q = _q->memory();
    std::byte *attn = _attn->memory(), *gate_up = _gate_up->memory(), *act = _act->memory();
    const std::vector<Layer> layers = layerPointers();

    // Per layer: norm, packed q|k|v projection, [bias + rope + append], attention, output projection accumulated into the
    // residual stream, norm, packed gate|up projection, activation, down projection accumulated into the stream.
    opEmbedding(x, a.tokens, _weights.in_embed->tensor->data(), T, hs, _meta.voc);
    for (size_t l = 0; l < _meta.nlayer; ++l) {
        const Layer &w = layers[l];
        opRmsNorm(h, x, w.attn_norm, T, hs);
        opLinear(qkv, h, w.qkv_w, T, qd + 2 * kd, hs);
        _cache->ropeAppendDev(l, q, qkv, w.qkv_b, a.seq32, a.pos32, T, _meta.nh, _meta.theta, _stream);
        if (decode_only) {
            _cache->decodeDev(l, attn, nullptr, q, a.seq_list, a.kv_lens, n_seqs, max_kv_len, _meta.nh, scale, _stream);
        } else {
            _cache->prefillDev(l, attn, q, a.seq_list, a.q_starts, a.kv_lens, n_seqs, T, max_q_len, max_kv_len, _meta.nh,
                               scale, _stream);
        }
        projectIntoStream(x, h, attn, w.o_w, T, hs, qd);
        opRmsNorm(h, x, w.mlp_norm, T, hs);
        opLinear(gate_up, h, w.gate_up_w, T, 2 * di, hs);
        opSwigluPacked(act, gate_up, T, di);
        projectIntoStream(x, h, act, w.down_w, T, hs, di);
    }
    // the last token of every sequence -> final norm -> vocabulary projection -> greedy choice
    const std::byte *last = x;
    if (!decode_only) {
        opEmbedding(_x_last->memory(), a.last_rows, x, n_seqs, hs, T);
        last = _x_last->memory();
    }
    opRmsNorm(_x_last->memory(), last, _weights.out_norm_w->tensor->data(), n_seqs, hs);
    opLinear(_logits->memory(), _x_last->memory(), _weights.out_embed->tensor->data(), n_seqs, _meta.voc, hs);
    opArgmax(a.next, _logits->memory(), n_seqs, _meta.voc);
    _last_n_seqs = n_seqs;
}

void Qwen2::step(const int32_t *seq_ids, const int32_t *n_tokens, size_t n_seqs, const int64_t *tokens, int64_t *next_out) {
    if (n_seqs == 0) {
        return;
    }
    if (seq_ids == nullptr || n_tokens == nullptr || tokens == nullptr || next_out == nullptr) {
        fail(LLAISYS_E_INVALID, "qwen2: null argument");
    }
    size_t T = 0, max_q = 0, max_kv = 0;
    for (size_t i = 0; i < n_seqs; ++i) {
        const size_t len = seqLen(seq_ids[i]);
        if (n_tokens[i] < 1) {
            fail(LLAISYS_E_INVALID, "qwen2: every sequence of a step needs at least one new token");
        }
        if (len + size_t(n_tokens[i]) > _max_tokens_per_seq) {
            fail(LLAISYS_E_INVALID, "qwen2: sequence would exceed the configured maximum length");
        }
        for (size_t j = 0; j < i; ++j) {
            if (seq_ids[j] == seq_ids[i]) {
                fail(LLAISYS_E_INVALID, "qwen2: a sequence appears twice in one step");
            }
        }
        T += size_t(n_tokens[i]);
        max_q = std::max(max_q, size_t(n_tokens[i]));
        max_kv = std::max(max_kv, len + size_t(n_tokens[i]));
    }
    for (size_t i = 0; i < T; ++i) {
        if (tokens[i] < 0 || size_t(tokens[i]) >= _meta.voc) {
            fail(LLAISYS_E_INVALID, "qwen2: token id out of range");
        }
    }
    for (size_t i = 0; i < n_seqs; ++i) {
        _cache->seqReserve(seq_ids[i], seqLen(seq_ids[i]) + size_t(n_tokens[i]));
    }
    enter();
    ensureWorkspace(T, n_seqs);
    const StepArrays a = carveStepArrays(T, n_seqs);
    // the same carving over a host image, then one copy
    _meta_host.assign(_meta_bytes, std::byte{0});
    std::byte *dev0 = _meta_block->memory(), *host0 = _meta_host.data();
    auto host = [&](auto *dev_ptr) { return reinterpret_cast<decltype(dev_ptr)>(host0 + (reinterpret_cast<std::byte *>(dev_ptr) - dev0)); };
    size_t row = 0;
    bool decode_only = true;
    host(a.q_starts)[0] = 0;
    for (size_t i = 0; i < n_seqs; ++i) {
        const size_t len = seqLen(seq_ids[i]), n = size_t(n_tokens[i]);
        decode_only = decode_only && n == 1;
        for (size_t t = 0; t < n; ++t, ++row) {
            host(a.tokens)[row] = tokens[row];
            host(a.pos64)[row] = int64_t(len + t);
            host(a.pos32)[row] = int32_t(len + t);
            host(a.seq32)[row] = seq_ids[i];
        }
        host(a.kv_lens)[i] = int32_t(len + n);
        host(a.seq_list)[i] = seq_ids[i];
        host(a.q_starts)[i + 1] = int32_t(row);
        host(a.last_rows)[i] = int64_t(row) - 1;
    }
    copyToDevice(dev0, host0, _meta_bytes);
    _cache->flush();
    bool replayed = false;
#ifdef ENABLE_NVIDIA_API
    if (_on_gpu && decode_only && _tp_world == 1) {
        // The launch-bound case (nine kernels per layer): replay the step as a graph. The graph is captured with the
        // cache's maximum length as the attention kernels' bound, so it is valid for every later step of this batch size.
        if (_step_graphs.size() <= n_seqs) {
            _step_graphs.resize(n_seqs + 1);
        }
        StepGraph &g = _step_graphs[n_seqs];
        if (g.exec != nullptr && g.generation != _generation) {
            kernels::graph_destroy(g.exec);
            g = StepGraph{};
        }
        if (g.exec == nullptr && g.seen && g.generation == _generation) {
            enter().synchronize();
            kernels::graph_capture_begin(_stream);
            try {
                forward(a, T, n_seqs, 1, _max_tokens_per_seq, true);
            } catch (...) {
                kernels::graph_destroy(kernels::graph_capture_end(_stream));
                throw;
            }
            g.exec = kernels::graph_capture_end(_stream);
        }
        if (g.exec != nullptr) {
            kernels::graph_launch(g.exec, _stream);
            _last_n_seqs = n_seqs;
            replayed = true;
        } else {
            g.seen = true;
            g.generation = _generation;
            max_kv = _max_tokens_per_seq; // the eager step sizes scratch for what the capture will ask for
        }
    }
#endif
    if (!replayed) {
        forward(a, T, n_seqs, max_q, max_kv, decode_only);
    }
    copyToHost(next_out, a.next, n_seqs * sizeof(int64_t));
    for (size_t i = 0, at = 0; i < n_seqs; ++i) {
        seqLen(seq_ids[i]) += size_t(n_tokens[i]);
        recordTokens(seq_ids[i], tokens + at, size_t(n_tokens[i]));
        at += size_t(n_tokens[i]);
    }
    checkKernels();
}

void Qwen2::decodeLoop(const int32_t *seq_ids, size_t n_seqs, const int64_t *first_tokens, size_t n_steps,
                       int64_t *tokens_out) {
    if (n_seqs == 0 || n_steps == 0) {
        return;
    }
    if (seq_ids == nullptr || first_tokens == nullptr || tokens_out == nullptr) {
        fail(LLAISYS_E_INVALID, "qwen2: null argument");
    }
    size_t max_kv = 0;
    for (size_t i = 0; i < n_seqs; ++i) {
        const size_t len = seqLen(seq_ids[i]);
        if (len + n_steps > _max_tokens_per_seq) {
            fail(LLAISYS_E_INVALID, "qwen2: sequence would exceed the configured maximum length");
        }
        if (first_tokens[i] < 0 || size_t(first_tokens[i]) >= _meta.voc) {
            fail(LLAISYS_E_INVALID, "qwen2: token id out of range");
        }
        max_kv = std::max(max_kv, len + n_steps);
    }
    for (size_t i = 0; i < n_seqs; ++i) {
        _cache->seqReserve(seq_ids[i], seqLen(seq_ids[i]) + n_steps); // every page of the loop, up front
    }
    auto &rt = enter();
    ensureWorkspace(n_seqs, n_seqs);
    const StepArrays a = carveStepArrays(n_seqs, n_seqs);
    _meta_host.assign(_meta_bytes, std::byte{0});
    std::byte *dev0 = _meta_block->memory(), *host0 = _meta_host.data();
    auto host = [&](auto *dev_ptr) { return reinterpret_cast<decltype(dev_ptr)>(host0 + (reinterpret_cast<std::byte *>(dev_ptr) - dev0)); };
    for (size_t i = 0; i < n_seqs; ++i) {
        const size_t len = seqLen(seq_ids[i]);
        host(a.tokens)[i] = first_tokens[i];
        host(a.pos64)[i] = int64_t(len);
        host(a.pos32)[i] = int32_t(len);
        host(a.seq32)[i] = seq_ids[i];
        host(a.kv_lens)[i] = int32_t(len + 1);
        host(a.seq_list)[i] = seq_ids[i];
        host(a.q_starts)[i] = int32_t(i);
        host(a.last_rows)[i] = int64_t(i);
    }
    host(a.q_starts)[n_seqs] = int32_t(n_seqs);
    copyToDevice(dev0, host0, _meta_bytes);
    _cache->flush();
    // the token log and the step counter the advance kernel writes through
    core::storage_t log = rt.allocateDeviceStorage(n_steps * n_seqs * sizeof(int64_t));
    core::storage_t counter = rt.allocateDeviceStorage(sizeof(int32_t));
    const int32_t zero = 0;
    copyToDevice(counter->memory(), &zero, sizeof(zero));
    auto *log_dev = reinterpret_cast<int64_t *>(log->memory());
    auto *counter_dev = reinterpret_cast<int32_t *>(counter->memory());

    auto one_step = [&]() {
        forward(a, n_seqs, n_seqs, 1, max_kv, true);
#ifdef ENABLE_NVIDIA_API
        if (_on_gpu) {
            kernels::advance_decode_state(_stream, a.tokens, a.next, a.pos64, a.pos32, a.kv_lens, log_dev, counter_dev,
                                          int(n_seqs));
            return;
        }
#endif
        int32_t &step = *counter_dev;
        for (size_t i = 0; i < n_seqs; ++i) {
            a.tokens[i] = a.next[i];
            log_dev[size_t(step) * n_seqs + i] = a.next[i];
            a.pos64[i] += 1;
            a.pos32[i] += 1;
            a.kv_lens[i] += 1;
        }
        ++step;
    };

    if (_on_gpu) {
#ifdef ENABLE_NVIDIA_API
        one_step(); // eager: sizes every lazily grown scratch before the capture
        size_t timed_steps = 0;
        float ms = 0.f;
        if (n_steps > 1) {
            rt.synchronize();
            kernels::graph_capture_begin(_stream);
            try {
                one_step();
            } catch (...) {
                kernels::graph_destroy(kernels::graph_capture_end(_stream));
                throw;
            }
            void *exec = kernels::graph_capture_end(_stream);
            void *e0 = kernels::event_create(), *e1 = kernels::event_create();
            kernels::event_record(e0, _stream);
            for (size_t s = 1; s < n_steps; ++s) {
                kernels::graph_launch(exec, _stream);
            }
            kernels::event_record(e1, _stream);
            ms = kernels::event_elapsed_ms(e0, e1);
            timed_steps = n_steps - 1;
            kernels::event_destroy(e0);
            kernels::event_destroy(e1);
            kernels::graph_destroy(exec);
        }
        _last_loop_ms = timed_steps ? double(ms) / double(timed_steps) : 0.0;
#endif
    } else {
        const auto t0 = std::chrono::steady_clock::now();
        for (size_t s = 0; s < n_steps; ++s) {
            one_step();
        }
        _last_loop_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / double(n_steps);
    }
    copyToHost(tokens_out, log_dev, n_steps * n_seqs * sizeof(int64_t));
    std::vector<int64_t> fed(n_steps);
    for (size_t i = 0; i < n_seqs; ++i) {
        seqLen(seq_ids[i]) += n_steps;
        fed[0] = first_tokens[i]; // step s consumed the token step s - 1 produced
        for (size_t st = 1; st < n_steps; ++st) {
            fed[st] = tokens_out[(st - 1) * n_seqs + i];
        }
        recordTokens(seq_ids[i], fed.data(), n_steps);
    }
    checkKernels();
}

// Error words of the kernels a step ran: the cache's (bad block-table entries, a wait that ran out in an attention
// kernel) and the projection kernel's.
void Qwen2::checkKernels() {
    _cache->check();
#ifdef ENABLE_NVIDIA_API
    if (_on_gpu) {
        const int status = kernels::linear_tc_status(_stream);
        if (status != 0) {
            fail(LLAISYS_E_KERNEL, "qwen2: the projection kernel reported error word " + std::to_string(status));
        }
    }
#endif
}

void Qwen2::lastLogits(float *out_host, size_t capacity_floats) {
    const size_t n = _last_n_seqs * _meta.voc;
    if (n == 0) {
        fail(LLAISYS_E_INVALID, "qwen2: no step has run yet");
    }
    if (out_host == nullptr || capacity_floats < n) {
        fail(LLAISYS_E_INVALID, "qwen2: logits buffer too small");
    }
    std::vector<std::byte> raw(n * _elem);
    copyToHost(raw.data(), _logits->memory(), raw.size());
    for (size_t i = 0; i < n; ++i) {
        switch (_meta.dtype) {
        case LLAISYS_DTYPE_F32:
            out_host[i] = reinterpret_cast<const float *>(raw.data())[i];
            break;
        case LLAISYS_DTYPE_F16:
            out_host[i] = utils::cast<float>(reinterpret_cast<const fp16_t *>(raw.data())[i]);
            break;
        default:
            out_host[i] = utils::cast<float>(reinterpret_cast<const bf16_t *>(raw.data())[i]);
            break;
        }
    }
}

} // namespace llaisys::models
