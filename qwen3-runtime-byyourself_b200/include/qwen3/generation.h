// The decisions of the generation loop, as plain host code: which requests may run, how they are split into
// batches that fit the cache, and - token by token - which sequences go on and why the others ended.  The loop
// that drives an engine with them (steps, sampling, callbacks) is the binding's; nothing here touches a GPU.
//
// Per sequence the rules are the reference's (src/generation/generator.cpp:249-323): the chosen token is
// recorded, a stop token ends the sequence and is recorded but not fed back (:294-301), the budget of new tokens
// ends it without a further step (:305-307), a budget of zero returns before any step (:258-260); an empty prompt
// is an error (:85-89), prompt + new tokens must fit the context (:163-184), stop ids must lie in the vocabulary
// (:186-195).  The reference generates one sequence at a time (:79-83); batches are this library's.
#pragma once

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace qwen3 {

class GenerationError : public std::invalid_argument {
public:
    using std::invalid_argument::invalid_argument;
};

enum class StopReason : int { Running = 0, MaxNewTokens = 1, StopToken = 2 };

// Throws a GenerationError that names the first request (or stop id) that cannot run.
inline void check_requests(const int64_t* prompt_lengths, int n_requests, int64_t max_new_tokens, int64_t max_seq_len,
                           const int32_t* stop_token_ids, int n_stops, int64_t vocab_size) {
    if (max_new_tokens < 0) throw GenerationError("max_new_tokens cannot be negative");
    for (int s = 0; s < n_stops; ++s)
        if (stop_token_ids[s] < 0 || stop_token_ids[s] >= vocab_size)
            throw GenerationError("stop token id " + std::to_string(stop_token_ids[s]) + " is outside the vocabulary");
    for (int i = 0; i < n_requests; ++i) {
        if (prompt_lengths[i] <= 0) throw GenerationError("request " + std::to_string(i) + ": the prompt is empty");
        if (prompt_lengths[i] + max_new_tokens > max_seq_len)
            throw GenerationError("request " + std::to_string(i) + ": " + std::to_string(prompt_lengths[i]) + " prompt tokens + " +
                                  std::to_string(max_new_tokens) + " new tokens exceed the context of " +
                                  std::to_string(max_seq_len));
    }
}

// Requests in order, split into batches whose worst-case need of pages (prompt + every new token) fits the
// cache, with at most `n_slots` (and, if positive, `batch_size`) requests each.  Returns the batch of each request.
inline std::vector<int> plan_batches(const int64_t* prompt_lengths, int n_requests, int64_t max_new_tokens, int64_t n_pages,
                                     int n_slots, int page_tokens, int batch_size) {
    if (page_tokens <= 0 || n_slots <= 0) throw GenerationError("a cache has at least one slot and pages of at least one token");
    std::vector<int> batch_of((size_t)n_requests);
    int batch = 0, in_batch = 0;
    int64_t used = 0;
    for (int i = 0; i < n_requests; ++i) {
        const int64_t need = (prompt_lengths[i] + max_new_tokens + page_tokens - 1) / page_tokens;
        if (need > n_pages)
            throw GenerationError("request " + std::to_string(i) + ": " + std::to_string(prompt_lengths[i]) + " prompt + " +
                                  std::to_string(max_new_tokens) + " new tokens need " + std::to_string(need) +
                                  " pages, the cache has " + std::to_string(n_pages));
        const bool full = in_batch >= n_slots || (batch_size > 0 && in_batch >= batch_size);
        if (in_batch > 0 && (full || used + need > n_pages)) {
            ++batch;
            in_batch = 0;
            used = 0;
        }
        batch_of[(size_t)i] = batch;
        ++in_batch;
        used += need;
    }
    return batch_of;
}

// What has been generated for the requests of one call, and who is still running.
class GenerationProgress {
public:
    GenerationProgress(int n_requests, int64_t max_new_tokens, const int32_t* stop_token_ids, int n_stops)
        : max_new_(max_new_tokens), stops_(stop_token_ids, stop_token_ids + n_stops), produced_((size_t)n_requests, 0),
          reason_((size_t)n_requests, max_new_tokens > 0 ? StopReason::Running : StopReason::MaxNewTokens) {
        if (n_requests < 0 || max_new_tokens < 0) throw GenerationError("a generation has no negative sizes");
        std::sort(stops_.begin(), stops_.end());
    }

    int n_requests() const { return (int)produced_.size(); }
    int64_t produced(int request) const { return produced_[at(request)]; }
    StopReason reason(int request) const { return reason_[at(request)]; }
    bool running(int request) const { return reason(request) == StopReason::Running; }

    // The token chosen for `request` is recorded; true if the sequence goes on (the token is fed back).
    bool record(int request, int32_t token) {
        const size_t r = at(request);
        if (reason_[r] != StopReason::Running) throw GenerationError("request " + std::to_string(request) + " has ended");
        ++produced_[r];
        if (std::binary_search(stops_.begin(), stops_.end(), token)) reason_[r] = StopReason::StopToken;
        else if (produced_[r] >= max_new_) reason_[r] = StopReason::MaxNewTokens;
        return reason_[r] == StopReason::Running;
    }

    // A loop that runs one step ahead of the host asks before the pending token is known: would the sequence
    // still have budget after it?  (A stop token among the pending ones then costs one step too many.)
    bool may_run_ahead(int request) const { return running(request) && produced_[at(request)] + 1 < max_new_; }

private:
    size_t at(int request) const {
        if (request < 0 || (size_t)request >= produced_.size()) throw GenerationError("no request " + std::to_string(request));
        return (size_t)request;
    }
    int64_t max_new_;
    std::vector<int32_t> stops_;
    std::vector<int64_t> produced_;
    std::vector<StopReason> reason_;
};

}  // namespace qwen3
