// Iteration-level ("continuous") batching over one Qwen2 model and its paged KV cache: requests join a queue at any
// time; every step() forms one batch out of the running requests -- one token for each request that is decoding, the
// next chunk of the prompt for each that is still prefilling -- runs it as ONE model step, and hands the unfinished
// requests back. A request is admitted when the pool can hold its prompt and everything it may generate, so a running
// request never runs out of pages; its prompt first takes whatever whole pages the prefix cache already holds.
// New code: the reference describes this service as future work (README.md:415-424).
#pragma once

#include "../models/qwen2.hpp"

#include <deque>
#include <vector>

namespace llaisys::serve {

struct EngineConfig {
    size_t max_batch = 64;           // requests in one step
    size_t max_tokens_per_step = 4096; // decode tokens + prefill chunk tokens in one step
    size_t prefill_chunk = 512;      // prompt tokens one request may contribute to a step
};

struct Event {
    int64_t request; // id returned by submit
    int64_t token;   // the token generated for it in this step
    int32_t finished; // 1 = this was its last token (length limit or end token)
    int32_t reserved;
};

class Engine : private models::ModelObserver {
public:
    Engine(models::Qwen2 &model, const EngineConfig &cfg);
    ~Engine();
    Engine(const Engine &) = delete;
    Engine &operator=(const Engine &) = delete;

    // Queues a request; -> its id. end_token < 0 = the model's own (meta.end_token).
    int64_t submit(const int64_t *prompt, size_t n_prompt, size_t max_new_tokens, int64_t end_token);
    // One iteration. Writes at most `cap` events (a step yields at most max_batch), -> how many.
    size_t step(Event *events, size_t cap);
    bool cancel(int64_t request);
    size_t numWaiting() const { return _waiting.size(); }
    size_t numRunning() const { return _running.size(); }
    // counters since creation
    size_t stepsRun() const { return _steps; }
    size_t promptTokensFromCache() const { return _cached_tokens; }
    size_t tokensComputed() const { return _computed_tokens; }

private:
    struct Request {
        int64_t id = 0;
        std::vector<int64_t> prompt;
        size_t max_new = 0;
        int64_t end_token = -1;
        int32_t seq = -1;
        size_t fed = 0;        // prompt tokens whose K/V exist (matched from the cache or computed)
        size_t generated = 0;
        int64_t last = 0;      // the token to feed next once the prompt is in
    };

    void admit();
    void finish(size_t running_index);
    void modelDestroyed() override; // the model went first: forget it, every later call fails cleanly
    models::Qwen2 &model();

    models::Qwen2 *_model_ptr;
    EngineConfig _cfg;
    std::deque<Request> _waiting;
    std::vector<Request> _running;
    int64_t _next_id = 1;
    size_t _steps = 0, _cached_tokens = 0, _computed_tokens = 0;
    // batch under construction (members, so that steps do not allocate)
    std::vector<int32_t> _seq_ids, _n_tokens, _owner;
    std::vector<int64_t> _tokens, _next;
};

} // namespace llaisys::serve
