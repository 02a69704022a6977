// qwen3/cache_book.h - the bookkeeping of the paged key/value cache on the host: slots, lengths,
// pages and layer groups.  No device memory is touched here; the storage lives elsewhere and is
// indexed by the page numbers this class hands out.
//
// A *slot* belongs to one sequence from its first step until the batch gives it back.  Keys and
// values live in *pages* of `page_tokens` tokens; a slot holds, for every layer group, a list of
// pages that covers its length.  Layers whose mixers ask the same of the cache form a *group* with
// a page pool of its own; a group that needs only a window of keys returns the pages that fell out
// of the window after each step.
//
// A step is three calls: reserve (all or nothing: a step that does not fit changes nothing), the
// launch, then commit (lengths advance once) or cancel (the launch failed: the pages go back).
//
// The reference keeps two dense [L, Bmax, Smax, nkv, d] tensors with one length per layer shared by
// all batch rows (src/model/kv_cache.cpp:55-74, include/qwen3/model/kv_cache.h:93-99); its
// append-only rule (:115-117) and capacity check (:119-123) are kept here per slot.
//
// Header-only C++17.  Errors are thrown as qwen3::CacheError / qwen3::CacheFull.
#pragma once

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace qwen3 {

struct CacheError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct CacheFull : CacheError {
    using CacheError::CacheError;
};

enum class GroupKind : int { Full = 0, Window = 1 };

// The pages of the layers that share one need.
class PageGroup {
public:
    PageGroup(GroupKind kind, int window, int n_pages, int n_slots, int pages_per_slot, int page_tokens)
        : kind_(kind), window_(window), n_pages_(n_pages), pages_per_slot_(pages_per_slot), page_tokens_(page_tokens),
          table_((size_t)n_slots * pages_per_slot, -1), first_live_(n_slots, 0) {
        free_.reserve(n_pages);
        for (int p = n_pages - 1; p >= 0; --p) free_.push_back(p);
    }

    int n_pages() const { return n_pages_; }
    int n_free() const { return (int)free_.size(); }
    GroupKind kind() const { return kind_; }
    int window() const { return window_; }
    const std::vector<int32_t>& free_pages() const { return free_; }
    // [n_slots, pages_per_slot] page numbers, -1 where none is held.
    int32_t* table() { return table_.data(); }
    const int32_t* table() const { return table_.data(); }
    const int32_t* row(int slot) const { return table_.data() + (size_t)slot * pages_per_slot_; }
    int64_t first_live(int slot) const { return first_live_[slot]; }

    int pages_needed(int64_t length_now, int64_t n_new) const { return (int)(pages_for(length_now + n_new) - pages_for(length_now)); }

    void extend(int slot, int64_t length_now, int64_t n_new) {
        int32_t* r = table_.data() + (size_t)slot * pages_per_slot_;
        for (int64_t i = pages_for(length_now); i < pages_for(length_now + n_new); ++i) {
            r[i] = free_.back();
            free_.pop_back();
        }
    }
    // Undo extend(slot, length_now, n_new).
    void shrink(int slot, int64_t length_now, int64_t n_new) {
        int32_t* r = table_.data() + (size_t)slot * pages_per_slot_;
        for (int64_t i = pages_for(length_now + n_new) - 1; i >= pages_for(length_now); --i)
            if (r[i] >= 0) {
                free_.push_back(r[i]);
                r[i] = -1;
            }
    }
    // Give back the pages that no later query of this sequence can read (window groups).
    void trim_window(int slot, int64_t length) {
        if (kind_ != GroupKind::Window) return;
        // a query at position >= length reads keys > length - window
        int64_t dead = (length - window_ + 1) / page_tokens_;
        if (length - window_ + 1 < 0) dead = 0;
        int32_t* r = table_.data() + (size_t)slot * pages_per_slot_;
        for (int64_t i = first_live_[slot]; i < dead; ++i)
            if (r[i] >= 0) {
                free_.push_back(r[i]);
                r[i] = -1;
            }
        if (dead > first_live_[slot]) first_live_[slot] = dead;
    }
    void release(int slot) {
        int32_t* r = table_.data() + (size_t)slot * pages_per_slot_;
        for (int i = 0; i < pages_per_slot_; ++i)
            if (r[i] >= 0) {
                free_.push_back(r[i]);
                r[i] = -1;
            }
        first_live_[slot] = 0;
    }

private:
    int64_t pages_for(int64_t tokens) const { return (tokens + page_tokens_ - 1) / page_tokens_; }

    GroupKind kind_;
    int window_, n_pages_, pages_per_slot_, page_tokens_;
    std::vector<int32_t> free_, table_;
    std::vector<int64_t> first_live_;
};

// What one layer group asks of the cache.
struct GroupNeed {
    GroupKind kind = GroupKind::Full;
    int window = 0;        // Window groups: the number of keys a query reads
};

class CacheBook {
public:
    // `max_tokens`: the most tokens that live sequences hold at any time, each sequence rounded up to whole
    // pages; `max_seq_len` bounds one sequence; `n_slots` <= 0: as many slots as pages.
    CacheBook(const std::vector<GroupNeed>& groups, int64_t max_tokens, int64_t max_seq_len, int n_slots = 0, int page_tokens = 64)
        : page_tokens_(page_tokens) {
        if (max_tokens <= 0 || max_seq_len <= 0 || page_tokens <= 0) throw std::invalid_argument("max_tokens, max_seq_len and page_tokens must be positive");
        n_pages_ = (int)((max_tokens + page_tokens - 1) / page_tokens);
        max_seq_len_ = std::min<int64_t>(max_seq_len, (int64_t)n_pages_ * page_tokens);
        pages_per_slot_ = (int)((max_seq_len_ + page_tokens - 1) / page_tokens);
        n_slots_ = n_slots > 0 ? n_slots : n_pages_;
        lengths_.assign(n_slots_, 0);
        held_.assign(n_slots_, 0);
        for (int s = n_slots_ - 1; s >= 0; --s) free_slots_.push_back(s);
        for (const GroupNeed& g : groups) {
            if (g.kind == GroupKind::Window && g.window <= 0) throw std::invalid_argument("a window group needs a positive window");
            groups_.emplace_back(g.kind, g.window, n_pages_, n_slots_, pages_per_slot_, page_tokens);
        }
    }

    int n_pages() const { return n_pages_; }
    int n_slots() const { return n_slots_; }
    int pages_per_slot() const { return pages_per_slot_; }
    int page_tokens() const { return page_tokens_; }
    int64_t max_seq_len() const { return max_seq_len_; }
    int n_groups() const { return (int)groups_.size(); }
    PageGroup& group(int g) { return groups_[g]; }
    const PageGroup& group(int g) const { return groups_[g]; }
    int n_free_slots() const { return (int)free_slots_.size(); }
    bool is_held(int slot) const { return slot >= 0 && slot < n_slots_ && held_[slot]; }
    int64_t length(int slot) const { return lengths_[slot]; }
    int64_t* lengths() { return lengths_.data(); }

    // A free slot for a sequence that starts now (length 0).
    int alloc_slot() {
        if (free_slots_.empty()) throw CacheFull("all " + std::to_string(n_slots_) + " slots are held");
        const int slot = free_slots_.back();
        free_slots_.pop_back();
        held_[slot] = 1;
        lengths_[slot] = 0;
        return slot;
    }
    // The sequence is finished: its slot and pages are given back.
    void free_slot(int slot) {
        if (!is_held(slot)) throw CacheError("slot " + std::to_string(slot) + " is not held (freed twice, or never handed out)");
        held_[slot] = 0;
        free_slots_.push_back(slot);
        for (PageGroup& g : groups_) g.release(slot);
        lengths_[slot] = 0;
    }

    // Make room for n_new[i] tokens on slots[i]; nothing changes if it cannot be done.
    void reserve(const int* slots, const int64_t* n_new, int n) {
        seen_.assign(n_slots_, 0);
        for (int i = 0; i < n; ++i) {
            const int slot = slots[i];
            if (!is_held(slot)) throw CacheError("slot " + std::to_string(slot) + " is not held");
            if (seen_[slot]) throw CacheError("slot " + std::to_string(slot) + " appears twice in one step");
            seen_[slot] = 1;
            if (n_new[i] <= 0) throw CacheError("slot " + std::to_string(slot) + ": a step needs at least one token");
            if (lengths_[slot] + n_new[i] > max_seq_len_)
                throw CacheFull("slot " + std::to_string(slot) + ": " + std::to_string(lengths_[slot]) + " + " + std::to_string(n_new[i]) +
                                " tokens exceed the sequence capacity " + std::to_string(max_seq_len_));
        }
        for (const PageGroup& g : groups_) {
            int64_t need = 0;
            for (int i = 0; i < n; ++i) need += g.pages_needed(lengths_[slots[i]], n_new[i]);
            if (need > g.n_free())
                throw CacheFull("the step needs " + std::to_string(need) + " pages of " + std::to_string(page_tokens_) + " tokens, " +
                                std::to_string(g.n_free()) + " are free (of " + std::to_string(g.n_pages()) + ")");
        }
        for (PageGroup& g : groups_)
            for (int i = 0; i < n; ++i) g.extend(slots[i], lengths_[slots[i]], n_new[i]);
    }
    // The step ran: lengths advance once, window groups return dead pages.
    void commit(const int* slots, const int64_t* n_new, int n) {
        for (int i = 0; i < n; ++i) {
            lengths_[slots[i]] += n_new[i];
            for (PageGroup& g : groups_) g.trim_window(slots[i], lengths_[slots[i]]);
        }
    }
    // The step did not run after all: the pages that reserve took for it go back, lengths stay.
    void cancel(const int* slots, const int64_t* n_new, int n) {
        for (PageGroup& g : groups_)
            for (int i = 0; i < n; ++i) g.shrink(slots[i], lengths_[slots[i]], n_new[i]);
    }
    // Pages in use in the fullest group: what counts against max_tokens.
    int pages_held() const {
        int most = 0;
        for (const PageGroup& g : groups_) most = std::max(most, g.n_pages() - g.n_free());
        return most;
    }

private:
    int page_tokens_, n_pages_ = 0, pages_per_slot_ = 0, n_slots_ = 0;
    int64_t max_seq_len_ = 0;
    std::vector<int64_t> lengths_;
    std::vector<char> held_, seen_;
    std::vector<int> free_slots_;
    std::vector<PageGroup> groups_;
};

}  // namespace qwen3
