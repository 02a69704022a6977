// A host program against the public headers (include/qwen3/cache_book.h, step_pack.h, generation.h): the checks of the Python
// suite's cache tests, made from C++ without any binding.  Prints "ok" and exits 0, or says what failed.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <set>
#include <vector>

#include "qwen3/cache_book.h"
#include "qwen3/generation.h"
#include "qwen3/step_pack.h"

#define CHECK(cond)                                                           \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::printf("%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                         \
        }                                                                     \
    } while (0)

template <typename E, typename F> bool throws(F&& f) {
    try {
        f();
    } catch (const E&) {
        return true;
    } catch (...) {
        return false;
    }
    return false;
}

static std::vector<int> held_pages(const qwen3::CacheBook& book, int group, int slot) {
    std::vector<int> out;
    const int32_t* row = book.group(group).row(slot);
    for (int p = 0; p < book.pages_per_slot(); ++p)
        if (row[p] >= 0) out.push_back(row[p]);
    return out;
}

int main() {
    using namespace qwen3;
    {   // lengths, pages, reuse, all-or-nothing reservation, cancel
        CacheBook book({GroupNeed{}}, 5 * 64, 4 * 64);
        CHECK(book.n_pages() == 5 && book.pages_per_slot() == 4 && book.n_slots() == 5);
        const int a = book.alloc_slot(), b = book.alloc_slot();
        int slots[2] = {a, b};
        int64_t n_new[2] = {70, 1};
        book.reserve(slots, n_new, 2);
        book.commit(slots, n_new, 2);
        CHECK(book.length(a) == 70 && book.length(b) == 1 && book.pages_held() == 3);
        const std::vector<int> before = held_pages(book, 0, a);
        int64_t big[2] = {130, 200};
        CHECK(throws<CacheFull>([&] { book.reserve(slots, big, 2); }));         // 2 + 3 more pages wanted, 2 free
        CHECK(held_pages(book, 0, a) == before && book.group(0).n_free() == 2);
        int twice[2] = {a, a};
        CHECK(throws<CacheError>([&] { book.reserve(twice, n_new, 2); }));
        int64_t more[1] = {60};
        book.reserve(slots, more, 1);                                            // a: 70 -> 130, one more page
        CHECK(book.group(0).n_free() == 1);
        book.cancel(slots, more, 1);
        CHECK(book.group(0).n_free() == 2 && held_pages(book, 0, a) == before && book.length(a) == 70);
        book.free_slot(a);
        CHECK(throws<CacheError>([&] { book.free_slot(a); }));
        CHECK(book.pages_held() == 1 && book.alloc_slot() == a && book.length(a) == 0);
    }
    {   // a window group gives back the pages no later query can read
        CacheBook book({GroupNeed{}, GroupNeed{GroupKind::Window, 70}}, 8 * 64, 8 * 64, 2);
        const int s = book.alloc_slot();
        int slots[1] = {s};
        int64_t n[1] = {300};
        book.reserve(slots, n, 1);
        book.commit(slots, n, 1);
        CHECK(held_pages(book, 0, s).size() == 5);
        CHECK(held_pages(book, 1, s).size() == 2);       // keys 231..299 and on: pages 3 and 4
        CHECK(book.group(1).row(s)[0] == -1 && book.group(1).row(s)[3] >= 0);
    }
    {   // a random schedule never loses or doubles a page
        std::mt19937 rng(0);
        CacheBook book({GroupNeed{}}, 40 * 64, 9 * 64, 8);
        std::vector<int> live;
        for (int it = 0; it < 3000; ++it) {
            const int action = rng() % 10;
            if (action < 2 && live.size() < 8) {
                live.push_back(book.alloc_slot());
            } else if (action < 3 && !live.empty()) {
                const size_t i = rng() % live.size();
                book.free_slot(live[i]);
                live.erase(live.begin() + i);
            } else if (!live.empty()) {
                std::vector<int> slots;
                std::vector<int64_t> n_new;
                for (int s : live)
                    if (rng() % 10 < 6) {
                        slots.push_back(s);
                        n_new.push_back(1 + rng() % 99);
                    }
                if (slots.empty()) continue;
                try {
                    book.reserve(slots.data(), n_new.data(), (int)slots.size());
                } catch (const CacheFull&) {
                    continue;
                }
                if (rng() % 100 < 15) book.cancel(slots.data(), n_new.data(), (int)slots.size());
                else book.commit(slots.data(), n_new.data(), (int)slots.size());
            }
            std::set<int> seen;
            size_t held = 0;
            for (int s : live)
                for (int p : held_pages(book, 0, s)) {
                    CHECK(seen.insert(p).second);                                 // held twice
                    ++held;
                }
            CHECK((int)held + book.group(0).n_free() == book.n_pages());        // lost
            for (int p : book.group(0).free_pages()) CHECK(seen.insert(p).second);
            for (int s : live) CHECK((int64_t)held_pages(book, 0, s).size() == (book.length(s) + 63) / 64);
        }
    }
    {   // the metadata of a step
        CacheBook book({GroupNeed{}}, 6 * 64, 3 * 64, 3);
        const int a = book.alloc_slot(), b = book.alloc_slot();
        int first[2] = {a, b};
        int64_t n0[2] = {65, 3};
        book.reserve(first, n0, 2);
        book.commit(first, n0, 2);
        int slots[2] = {b, a};
        int64_t n_new[2] = {2, 1};
        book.reserve(slots, n_new, 2);
        const int32_t ids[3] = {7, 8, 9}, want[2] = {1, 2};
        StepLayout lay(3, 2, 2, book.n_groups(), book.pages_per_slot());
        std::vector<int32_t> out(lay.total, -7);
        pack_step(book, lay, slots, n_new, 2, ids, want, 2, out.data());
        CHECK(out[lay.token_ids] == 7 && out[lay.token_ids + 2] == 9);
        CHECK(out[lay.token_seq] == 0 && out[lay.token_seq + 1] == 0 && out[lay.token_seq + 2] == 1);
        CHECK(out[lay.token_pos] == 3 && out[lay.token_pos + 1] == 4 && out[lay.token_pos + 2] == 65);
        CHECK(out[lay.seq_slots] == b && out[lay.seq_slots + 1] == a);
        CHECK(out[lay.seq_start] == 0 && out[lay.seq_start + 1] == 2 && out[lay.seq_start + 2] == 3);
        CHECK(out[lay.seq_pos0] == 3 && out[lay.seq_pos0 + 1] == 65);
        CHECK(out[lay.want_rows] == 1 && out[lay.want_rows + 1] == 2);
        for (int p = 0; p < book.pages_per_slot(); ++p) {
            CHECK(out[lay.tables[0] + p] == book.group(0).row(b)[p]);
            CHECK(out[lay.tables[0] + book.pages_per_slot() + p] == book.group(0).row(a)[p]);
        }
        book.commit(slots, n_new, 2);
        // a decode step of four rows, two of them padding
        StepLayout dl(4, 4, 4, book.n_groups(), book.pages_per_slot());
        std::vector<int32_t> d(dl.total, -7);
        const int32_t next[2] = {11, 12};
        int live[2] = {a, b};
        pack_decode_step(book, dl, 4, live, 2, next, d.data());
        CHECK(d[dl.token_ids] == 11 && d[dl.token_ids + 1] == 12 && d[dl.token_ids + 2] == 0);
        CHECK(d[dl.token_pos] == 66 && d[dl.token_pos + 1] == 5 && d[dl.token_pos + 3] == 0);
        CHECK(d[dl.seq_slots + 2] == book.n_slots() && d[dl.tables[0] + 3 * book.pages_per_slot()] == book.n_pages());
        CHECK(d[dl.seq_start + 4] == 4 && d[dl.want_rows + 3] == 3);
    }
    // ---- the generation loop's decisions
    {
        const int64_t lengths[8] = {100, 20, 65, 64, 1, 1, 1, 200};
        // 10 new tokens each: pages needed 2 1 2 2 1 1 1 4; a cache of 4 pages and 3 slots
        const std::vector<int> plan = plan_batches(lengths, 8, 10, 4, 3, 64, 0);
        const int want[8] = {0, 0, 1, 1, 2, 2, 2, 3};
        for (int i = 0; i < 8; ++i) CHECK(plan[i] == want[i]);
        const std::vector<int> by_two = plan_batches(lengths, 5, 1, 100, 100, 64, 2);
        CHECK(by_two[0] == 0 && by_two[1] == 0 && by_two[2] == 1 && by_two[3] == 1 && by_two[4] == 2);
        CHECK(throws<GenerationError>([&] { plan_batches(lengths, 8, 100, 4, 3, 64, 0); }));        // 200 + 100 tokens: 5 pages
        const int32_t stops[2] = {7, 3};
        check_requests(lengths, 8, 10, 210, stops, 2, 50);
        CHECK(throws<GenerationError>([&] { check_requests(lengths, 8, 11, 210, stops, 2, 50); }));   // 200 + 11 > 210
        CHECK(throws<GenerationError>([&] { check_requests(lengths, 8, 10, 210, stops, 2, 7); }));    // stop id 7 of 7
        const int64_t empty[2] = {4, 0};
        CHECK(throws<GenerationError>([&] { check_requests(empty, 2, 1, 210, stops, 0, 50); }));
        CHECK(throws<GenerationError>([&] { check_requests(lengths, 8, -1, 210, stops, 0, 50); }));

        GenerationProgress p(3, 3, stops, 2);
        CHECK(p.running(0) && p.may_run_ahead(0));
        CHECK(p.record(0, 5) && p.record(0, 6));                       // two of three: goes on
        CHECK(!p.may_run_ahead(0));                                    // whatever the pending token is, it is the last
        CHECK(!p.record(0, 9) && p.reason(0) == StopReason::MaxNewTokens && p.produced(0) == 3);
        CHECK(!p.record(1, 3) && p.reason(1) == StopReason::StopToken && p.produced(1) == 1);      // the stop token counts
        CHECK(p.record(2, 4) && !p.record(2, 7) && p.reason(2) == StopReason::StopToken);
        CHECK(throws<GenerationError>([&] { p.record(1, 5); }));      // it has ended
        CHECK(throws<GenerationError>([&] { p.record(3, 5); }));      // no such request
        GenerationProgress none(2, 0, stops, 0);
        CHECK(!none.running(0) && none.reason(1) == StopReason::MaxNewTokens && !none.may_run_ahead(0));
    }
    std::printf("ok\n");
    return 0;
}
