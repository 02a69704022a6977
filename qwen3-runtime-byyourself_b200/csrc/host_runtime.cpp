// The C face of the host runtime (include/qwen3/cache_book.h, step_pack.h, generation.h) for bindings:
// the cache book behind an opaque handle, the step packer, the generation loop's decisions, and the last
// error's text.  Every call returns 0, or 1 (misuse of the cache), 2 (the cache is full), 4 (a request that
// cannot be generated), 3 (anything else); q3_host_last_error() then gives the message of the calling
// thread's last failure.
#include <cstring>
#include <string>

#include "../include/qwen3/cache_book.h"
#include "../include/qwen3/generation.h"
#include "../include/qwen3/step_pack.h"

#define Q3_HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;

template <typename F> int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const qwen3::CacheFull& e) {
        g_error = e.what();
        return 2;
    } catch (const qwen3::CacheError& e) {
        g_error = e.what();
        return 1;
    } catch (const qwen3::GenerationError& e) {
        g_error = e.what();
        return 4;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 3;
    }
}

qwen3::CacheBook* book_of(void* h) { return static_cast<qwen3::CacheBook*>(h); }
qwen3::GenerationProgress* progress_of(void* h) { return static_cast<qwen3::GenerationProgress*>(h); }

}  // namespace

Q3_HOST_EXPORT const char* q3_host_last_error() { return g_error.c_str(); }

// kinds[g]: 0 = every key, 1 = a window of windows[g] keys.
Q3_HOST_EXPORT int q3_book_create(const int* kinds, const int* windows, int n_groups, int64_t max_tokens, int64_t max_seq_len,
                                  int n_slots, int page_tokens, void** out) {
    return guarded([&] {
        std::vector<qwen3::GroupNeed> needs(n_groups);
        for (int g = 0; g < n_groups; ++g) {
            needs[g].kind = kinds[g] ? qwen3::GroupKind::Window : qwen3::GroupKind::Full;
            needs[g].window = windows[g];
        }
        *out = new qwen3::CacheBook(needs, max_tokens, max_seq_len, n_slots, page_tokens);
    });
}
Q3_HOST_EXPORT void q3_book_destroy(void* h) { delete book_of(h); }
// info: n_pages, n_slots, pages_per_slot, page_tokens, n_groups; returns max_seq_len.
Q3_HOST_EXPORT int64_t q3_book_info(void* h, int* info) {
    const qwen3::CacheBook& b = *book_of(h);
    info[0] = b.n_pages(); info[1] = b.n_slots(); info[2] = b.pages_per_slot(); info[3] = b.page_tokens(); info[4] = b.n_groups();
    return b.max_seq_len();
}
Q3_HOST_EXPORT int q3_book_alloc_slot(void* h, int* slot) { return guarded([&] { *slot = book_of(h)->alloc_slot(); }); }
Q3_HOST_EXPORT int q3_book_free_slot(void* h, int slot) { return guarded([&] { book_of(h)->free_slot(slot); }); }
Q3_HOST_EXPORT int q3_book_reserve(void* h, const int* slots, const int64_t* n_new, int n) {
    return guarded([&] { book_of(h)->reserve(slots, n_new, n); });
}
Q3_HOST_EXPORT int q3_book_commit(void* h, const int* slots, const int64_t* n_new, int n) {
    return guarded([&] { book_of(h)->commit(slots, n_new, n); });
}
Q3_HOST_EXPORT int q3_book_cancel(void* h, const int* slots, const int64_t* n_new, int n) {
    return guarded([&] { book_of(h)->cancel(slots, n_new, n); });
}
Q3_HOST_EXPORT int64_t* q3_book_lengths(void* h) { return book_of(h)->lengths(); }
Q3_HOST_EXPORT int q3_book_is_held(void* h, int slot) { return book_of(h)->is_held(slot) ? 1 : 0; }
Q3_HOST_EXPORT int q3_book_free_slots(void* h) { return book_of(h)->n_free_slots(); }
Q3_HOST_EXPORT int q3_book_pages_held(void* h) { return book_of(h)->pages_held(); }
Q3_HOST_EXPORT int32_t* q3_book_table(void* h, int group) { return book_of(h)->group(group).table(); }
Q3_HOST_EXPORT int q3_book_free_pages(void* h, int group, int32_t* out) {      // out: n_pages elements at most; returns the count
    const std::vector<int32_t>& f = book_of(h)->group(group).free_pages();
    if (out != nullptr && !f.empty()) std::memcpy(out, f.data(), f.size() * sizeof(int32_t));
    return (int)f.size();
}

// The metadata of a step into `out` (see include/qwen3/step_pack.h); `offsets` receives the section offsets
// token_ids, token_seq, token_pos, seq_slots, seq_start, seq_pos0, want_rows, then one per group; returns the total.
Q3_HOST_EXPORT int q3_step_layout(int n_tokens, int n_seqs, int n_want, int n_groups, int pages_per_slot, int* offsets) {
    const qwen3::StepLayout lay(n_tokens, n_seqs, n_want, n_groups, pages_per_slot);
    if (offsets != nullptr) {
        const int fixed[7] = {lay.token_ids, lay.token_seq, lay.token_pos, lay.seq_slots, lay.seq_start, lay.seq_pos0, lay.want_rows};
        std::memcpy(offsets, fixed, sizeof(fixed));
        for (int g = 0; g < n_groups; ++g) offsets[7 + g] = lay.tables[g];
    }
    return lay.total;
}
Q3_HOST_EXPORT int q3_pack_step(void* h, const int* slots, const int64_t* n_new, int n_seqs, const int32_t* token_ids, int64_t n_tokens,
                                const int32_t* want_rows, int n_want, int32_t* out) {
    return guarded([&] {
        const qwen3::CacheBook& b = *book_of(h);
        const qwen3::StepLayout lay((int)n_tokens, n_seqs, n_want, b.n_groups(), b.pages_per_slot());
        qwen3::pack_step(b, lay, slots, n_new, n_seqs, token_ids, want_rows, n_want, out);
    });
}
Q3_HOST_EXPORT int q3_pack_decode_step(void* h, int rows, const int* slots, int n_live, const int32_t* token_ids, int32_t* out) {
    return guarded([&] {
        const qwen3::CacheBook& b = *book_of(h);
        const qwen3::StepLayout lay(rows, rows, rows, b.n_groups(), b.pages_per_slot());
        qwen3::pack_decode_step(b, lay, rows, slots, n_live, token_ids, out);
    });
}

// ---- the generation loop's decisions (include/qwen3/generation.h)
Q3_HOST_EXPORT int q3_generation_check(const int64_t* prompt_lengths, int n_requests, int64_t max_new_tokens, int64_t max_seq_len,
                                       const int32_t* stop_token_ids, int n_stops, int64_t vocab_size) {
    return guarded([&] { qwen3::check_requests(prompt_lengths, n_requests, max_new_tokens, max_seq_len, stop_token_ids, n_stops, vocab_size); });
}
// batch_of[i]: the batch (0, 1, ..) of request i; batch_size 0 = no limit beside slots and pages.
Q3_HOST_EXPORT int q3_generation_plan_batches(const int64_t* prompt_lengths, int n_requests, int64_t max_new_tokens, int64_t n_pages,
                                              int n_slots, int page_tokens, int batch_size, int* batch_of) {
    return guarded([&] {
        const std::vector<int> plan = qwen3::plan_batches(prompt_lengths, n_requests, max_new_tokens, n_pages, n_slots, page_tokens, batch_size);
        if (!plan.empty()) std::memcpy(batch_of, plan.data(), plan.size() * sizeof(int));
    });
}
Q3_HOST_EXPORT int q3_progress_create(int n_requests, int64_t max_new_tokens, const int32_t* stop_token_ids, int n_stops, void** out) {
    return guarded([&] { *out = new qwen3::GenerationProgress(n_requests, max_new_tokens, stop_token_ids, n_stops); });
}
Q3_HOST_EXPORT void q3_progress_destroy(void* h) { delete progress_of(h); }
// The tokens chosen in one step: goes_on[k] = 1 if requests[k] continues with tokens[k] fed back, else 0 and
// reasons[k] says why it ended (1: its budget of new tokens, 2: a stop token).
Q3_HOST_EXPORT int q3_progress_record(void* h, const int* requests, const int32_t* tokens, int n, int* goes_on, int* reasons) {
    return guarded([&] {
        qwen3::GenerationProgress& p = *progress_of(h);
        for (int k = 0; k < n; ++k) {
            goes_on[k] = p.record(requests[k], tokens[k]) ? 1 : 0;
            reasons[k] = (int)p.reason(requests[k]);
        }
    });
}
Q3_HOST_EXPORT int q3_progress_may_run_ahead(void* h, int request) {
    try {
        return progress_of(h)->may_run_ahead(request) ? 1 : 0;
    } catch (const std::exception&) {
        return 0;
    }
}
