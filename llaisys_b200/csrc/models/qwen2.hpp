// Qwen2 decoder (RMSNorm, GQA attention with q/k/v biases and half-split RoPE, SwiGLU MLP, untied output embedding)
// on the library's operators and the paged KV cache. The reference declares this model's C API and leaves it
// unimplemented (include/llaisys/models/qwen2.h:7-40; python/llaisys/models/qwen2.py:11-33 is a stub).
//
// All state of a forward pass lives on the model's device: activations in a workspace sized for the largest batch
// seen, per-step index arrays (tokens, positions, sequence rows, lengths) in one staging block. A decode loop keeps
// even the loop-carried state there: the chosen tokens feed the next step's embedding lookup, positions and lengths
// are advanced by a kernel, and on NVIDIA one step is captured as a CUDA graph and replayed.
#pragma once

#include "../capi/handles.hpp"
#include "../comm/collective.hpp"
#include "../kv/paged_kv.hpp"
#include "llaisys/models/qwen2.h"

#include <memory>
#include <vector>

namespace llaisys::models {

// Objects that borrow a model (a serving engine) hear about its destruction instead of touching freed memory when the
// owner destroys the two in the wrong order.
struct ModelObserver {
    virtual void modelDestroyed() = 0;

protected:
    ~ModelObserver() = default;
};

class Qwen2 {
public:
    void addObserver(ModelObserver *o) { _observers.push_back(o); }
    void removeObserver(ModelObserver *o) {
        for (size_t i = 0; i < _observers.size(); ++i) {
            if (_observers[i] == o) {
                _observers.erase(_observers.begin() + ptrdiff_t(i));
                return;
            }
        }
    }

    // tp_rank / tp_world: tensor parallelism by heads. Rank r holds query heads [r nh/W, (r+1) nh/W), the KV heads they
    // use, and rows [r di/W, (r+1) di/W) of the MLP; the output and down projections produce partial sums that one
    // all-reduce each turns into the full activation (set the collective before the first step). Embeddings, norms and
    // the vocabulary projection are replicated, so every rank computes the same logits and tokens.
    Qwen2(const LlaisysQwen2Meta &meta, llaisysDeviceType_t device, int device_id, int tp_rank = 0, int tp_world = 1);
    void setCollective(std::unique_ptr<comm::Collective> c);
    llaisysDeviceType_t deviceType() const { return _device; }
    int deviceId() const { return _device_id; }
    int tpRank() const { return _tp_rank; }
    int tpWorld() const { return _tp_world; }
    ~Qwen2();
    Qwen2(const Qwen2 &) = delete;
    Qwen2 &operator=(const Qwen2 &) = delete;

    LlaisysQwen2Weights *weights() { return &_weights; }
    const LlaisysQwen2Meta &meta() const { return _meta; } // this rank's share: nh, nkvh and di are per-rank under TP

    void configureCache(size_t max_seqs, size_t max_tokens);
    int32_t seqAdd();
    // New sequence that starts from the cached K/V of the longest published whole-page prefix of tokens[0, n) that leaves
    // at least one token to run; *matched = tokens already covered (feed tokens[*matched, n) to step()).
    int32_t seqAddWithPrefix(const int64_t *tokens, size_t n, size_t *matched);
    void seqReserve(int32_t seq, size_t n_tokens); // pages for n_tokens now, so that later steps cannot run out
    size_t seqLength(int32_t seq) { return seqLen(seq); }
    size_t freePages() const { return _cache ? _cache->numFreePages() : 0; }
    size_t maxTokensPerSeq() const { return _max_tokens_per_seq; }
    void seqFree(int32_t seq);
    void reset();
    int64_t infer(const int64_t *tokens, size_t n);
    void step(const int32_t *seq_ids, const int32_t *n_tokens, size_t n_seqs, const int64_t *tokens, int64_t *next_out);
    void decodeLoop(const int32_t *seq_ids, size_t n_seqs, const int64_t *first_tokens, size_t n_steps,
                    int64_t *tokens_out);
    void lastLogits(float *out_host, size_t capacity_floats);
    double lastLoopMs() const { return _last_loop_ms; }

private:
    // q|k|v and gate|up live packed in one matrix each (one projection launch instead of three / two); the handles the
    // caller loads through are row slices of the packed tensors
    struct Layer {
        const std::byte *attn_norm, *qkv_w, *qkv_b, *o_w, *mlp_norm, *gate_up_w, *down_w;
    };
    // device pointers of one step's index arrays (all inside _meta_block)
    struct StepArrays {
        int64_t *tokens = nullptr, *pos64 = nullptr, *last_rows = nullptr, *next = nullptr;
        int32_t *seq32 = nullptr, *pos32 = nullptr, *kv_lens = nullptr, *q_starts = nullptr, *seq_list = nullptr;
    };

    core::Runtime &enter() const;
    llaisysTensor_t wrap(tensor_t t);
    llaisysTensor_t makeWeight(const std::vector<size_t> &shape);
    std::vector<Layer> layerPointers() const;
    void ensureWorkspace(size_t n_tokens, size_t n_seqs);
    StepArrays carveStepArrays(size_t n_tokens, size_t n_seqs);
    size_t &seqLen(int32_t seq);
    // the network itself: activations for n_tokens rows -> logits and greedy tokens for n_seqs rows
    void forward(const StepArrays &a, size_t n_tokens, size_t n_seqs, size_t max_q_len, size_t max_kv_len, bool decode_only);

    // operator shims: CPU loops or CUDA launches on the runtime stream, on raw device pointers
    void opEmbedding(void *out, const int64_t *idx, const void *w, size_t n, size_t d, size_t vocab);
    void opLinear(void *out, const void *in, const void *w, size_t m, size_t n, size_t k, bool accumulate = false);
    void opRmsNorm(void *out, const void *in, const void *w, size_t rows, size_t d);
    void opSwigluPacked(void *out, const void *gate_up, size_t rows, size_t di);
    void opAdd(void *c, const void *a, const void *b, size_t n);
    // x += in . w^T, through an all-reduce of the partial product when the model is sharded
    void projectIntoStream(void *x, void *tmp, const void *in, const void *w, size_t m, size_t n, size_t k);
    void opArgmax(int64_t *idx, const void *vals, size_t rows, size_t n);
    void checkKernels();
    void copyToDevice(void *dst, const void *src, size_t bytes);
    void copyToHost(void *dst, const void *src, size_t bytes);

    LlaisysQwen2Meta _meta; // per-rank dimensions
    int _tp_rank = 0, _tp_world = 1;
    std::unique_ptr<comm::Collective> _tp;
    llaisysDeviceType_t _device;
    int _device_id;
    size_t _elem = 0;
    bool _on_gpu = false;
    llaisysStream_t _stream = nullptr;

    LlaisysQwen2Weights _weights{};
    std::vector<llaisysTensor_t> _all_weights; // owns every handle in _weights
    std::vector<llaisysTensor_t> _per_layer[12];
    std::vector<tensor_t> _qkv_w, _qkv_b, _gate_up_w; // packed per-layer matrices behind the q/k/v and gate/up handles

    std::unique_ptr<kv::PagedKV> _cache;
    size_t _max_tokens_per_seq = 0;
    std::vector<size_t> _seq_len; // by sequence id; SIZE_MAX = not live
    std::vector<std::vector<int64_t>> _seq_tokens; // ids of the tokens each sequence holds (keys of the prefix cache)
    void recordTokens(int32_t seq, const int64_t *tokens, size_t n);
    int32_t _implicit_seq = -1;

    // workspace
    core::storage_t _x, _h, _qkv, _q, _attn, _gate_up, _act, _x_last, _logits, _meta_block, _argmax_scratch;
    size_t _ws_tokens = 0, _ws_seqs = 0, _meta_bytes = 0;
    std::vector<std::byte> _meta_host;
    // Decode steps of step() (every sequence one token) replayed as CUDA graphs, one per batch size: the first step of
    // a size runs eagerly (it sizes scratch), the second is captured, later ones are replayed. A graph is dropped when
    // a buffer it points into is reallocated (generation) or the cache is reconfigured.
    struct StepGraph {
        void *exec = nullptr;
        uint64_t generation = 0;
        bool seen = false;
    };
    std::vector<StepGraph> _step_graphs; // by n_seqs
    uint64_t _generation = 1;
    void dropStepGraphs();
    std::vector<ModelObserver *> _observers;
    size_t _last_n_seqs = 0;
    double _last_loop_ms = 0.0;
};

} // namespace llaisys::models
