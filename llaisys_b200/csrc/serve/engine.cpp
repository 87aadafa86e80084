#include "engine.hpp"

#include "llaisys/paged_kv.h"

#include <algorithm>

namespace llaisys::serve {

namespace {
[[noreturn]] void fail(int code, const std::string &msg) { throw kv::StatusError(code, msg); }
constexpr size_t kPage = 16;
} // namespace

Engine::Engine(models::Qwen2 &model, const EngineConfig &cfg) : _model_ptr(&model), _cfg(cfg) {
    if (cfg.max_batch == 0 || cfg.max_tokens_per_step == 0 || cfg.prefill_chunk == 0) {
        fail(LLAISYS_E_INVALID, "engine: limits must be positive");
    }
    if (model.maxTokensPerSeq() == 0) {
        fail(LLAISYS_E_INVALID, "engine: configure the model's cache first (llaisysQwen2ModelConfigureCache)");
    }
    model.addObserver(this);
}

Engine::~Engine() {
    if (_model_ptr == nullptr) {
        return;
    }
    _model_ptr->removeObserver(this);
    for (Request &r : _running) {
        try {
            _model_ptr->seqFree(r.seq);
        } catch (...) {
        }
    }
}

void Engine::modelDestroyed() {
    _model_ptr = nullptr;
    _running.clear();
    _waiting.clear();
}

models::Qwen2 &Engine::model() {
    if (_model_ptr == nullptr) {
        fail(LLAISYS_E_INVALID, "engine: its model has been destroyed");
    }
    return *_model_ptr;
}

int64_t Engine::submit(const int64_t *prompt, size_t n_prompt, size_t max_new_tokens, int64_t end_token) {
    if (prompt == nullptr || n_prompt == 0) {
        fail(LLAISYS_E_INVALID, "engine: a request needs at least one prompt token");
    }
    if (max_new_tokens == 0) {
        fail(LLAISYS_E_INVALID, "engine: max_new_tokens must be positive");
    }
    // the last generated token is returned, never fed back: K/V are needed for prompt + max_new - 1 tokens
    if (n_prompt + max_new_tokens - 1 > model().maxTokensPerSeq()) {
        fail(LLAISYS_E_INVALID, "engine: prompt + max_new_tokens exceed the cache's maximum sequence length");
    }
    for (size_t i = 0; i < n_prompt; ++i) {
        if (prompt[i] < 0 || size_t(prompt[i]) >= model().meta().voc) {
            fail(LLAISYS_E_INVALID, "engine: token id out of range");
        }
    }
    Request r;
    r.id = _next_id++;
    r.prompt.assign(prompt, prompt + n_prompt);
    r.max_new = max_new_tokens;
    r.end_token = end_token < 0 ? model().meta().end_token : end_token;
    _waiting.push_back(std::move(r));
    return _waiting.back().id;
}

bool Engine::cancel(int64_t request) {
    for (auto it = _waiting.begin(); it != _waiting.end(); ++it) {
        if (it->id == request) {
            _waiting.erase(it);
            return true;
        }
    }
    for (size_t i = 0; i < _running.size(); ++i) {
        if (_running[i].id == request) {
            finish(i);
            return true;
        }
    }
    return false;
}

void Engine::finish(size_t running_index) {
    model().seqFree(_running[running_index].seq);
    _running.erase(_running.begin() + ptrdiff_t(running_index));
}

// First come, first served: the head of the queue is admitted as soon as a batch slot, a sequence slot and the pages
// for its whole life are there; nobody overtakes it (no starvation of long requests).
void Engine::admit() {
    while (!_waiting.empty() && _running.size() < _cfg.max_batch) {
        Request &r = _waiting.front();
        const size_t need_tokens = r.prompt.size() + r.max_new - 1;
        size_t matched = 0;
        int32_t seq = -1;
        try {
            seq = model().seqAddWithPrefix(r.prompt.data(), r.prompt.size(), &matched);
        } catch (const kv::StatusError &e) {
            if (e.code == LLAISYS_E_NO_SEQ) {
                return; // every sequence slot is taken: wait for a request to finish
            }
            throw;
        }
        try {
            model().seqReserve(seq, need_tokens);
        } catch (const kv::StatusError &e) {
            model().seqFree(seq);
            if (e.code == LLAISYS_E_NO_PAGES) {
                if (_running.empty()) {
                    fail(LLAISYS_E_NO_PAGES, "engine: request " + std::to_string(r.id) + " needs " +
                                                 std::to_string((need_tokens + kPage - 1) / kPage) +
                                                 " pages, more than the whole pool can give");
                }
                return; // wait for pages
            }
            throw;
        }
        r.seq = seq;
        r.fed = matched;
        _cached_tokens += matched;
        _running.push_back(std::move(r));
        _waiting.pop_front();
    }
}

size_t Engine::step(Event *events, size_t cap) {
    admit();
    if (_running.empty()) {
        return 0;
    }
    if (events == nullptr || cap < std::min(_running.size(), _cfg.max_batch)) {
        fail(LLAISYS_E_INVALID, "engine: the event buffer must hold one event per running request");
    }
    // Decode tokens first (they are what users wait for), then prompt chunks with what is left of the step's budget.
    _seq_ids.clear();
    _n_tokens.clear();
    _owner.clear();
    _tokens.clear();
    // Both scans start one request further on every step: with a budget smaller than the number of running requests
    // the ones that go without a token change from step to step, so every request keeps making progress.
    // While a prompt is still being fed, a share of the budget (a chunk, at most half) is kept back for it: decoding
    // requests alone can never take all of a small budget step after step.
    size_t budget = _cfg.max_tokens_per_step;
    const size_t n_run = _running.size(), first = _steps % n_run;
    const bool prompts_pending =
        std::any_of(_running.begin(), _running.end(), [](const Request &r) { return r.fed < r.prompt.size(); });
    const size_t kept_back = prompts_pending ? std::max<size_t>(1, std::min(_cfg.prefill_chunk, budget / 2)) : 0;
    const size_t decode_budget = budget > kept_back ? budget - kept_back : (prompts_pending ? 0 : budget);
    size_t decoded = 0;
    for (size_t k = 0; k < n_run && decoded < decode_budget; ++k) {
        const size_t i = (first + k) % n_run;
        Request &r = _running[i];
        if (r.fed == r.prompt.size()) {
            ++decoded;
            _seq_ids.push_back(r.seq);
            _n_tokens.push_back(1);
            _owner.push_back(int32_t(i));
            _tokens.push_back(r.last);
            --budget;
        }
    }
    for (size_t k = 0; k < n_run && budget > 0; ++k) {
        const size_t i = (first + k) % n_run;
        Request &r = _running[i];
        if (r.fed < r.prompt.size()) {
            const size_t n = std::min({_cfg.prefill_chunk, r.prompt.size() - r.fed, budget});
            _seq_ids.push_back(r.seq);
            _n_tokens.push_back(int32_t(n));
            _owner.push_back(int32_t(i));
            _tokens.insert(_tokens.end(), r.prompt.begin() + ptrdiff_t(r.fed), r.prompt.begin() + ptrdiff_t(r.fed + n));
            budget -= n;
        }
    }
    _next.assign(_seq_ids.size(), 0);
    model().step(_seq_ids.data(), _n_tokens.data(), _seq_ids.size(), _tokens.data(), _next.data());
    ++_steps;
    _computed_tokens += _tokens.size();

    size_t n_events = 0;
    std::vector<size_t> done;
    for (size_t b = 0; b < _seq_ids.size(); ++b) {
        Request &r = _running[size_t(_owner[b])];
        if (r.fed < r.prompt.size()) {
            r.fed += size_t(_n_tokens[b]);
            if (r.fed < r.prompt.size()) {
                continue; // mid-prompt chunk: its "next token" means nothing
            }
        }
        r.last = _next[b];
        ++r.generated;
        const bool finished = r.generated >= r.max_new || r.last == r.end_token;
        events[n_events++] = Event{r.id, r.last, finished ? 1 : 0, 0};
        if (finished) {
            done.push_back(size_t(_owner[b]));
        }
    }
    std::sort(done.rbegin(), done.rend()); // erase from the back so that indices stay valid
    for (size_t idx : done) {
        finish(idx);
    }
    return n_events;
}

} // namespace llaisys::serve
