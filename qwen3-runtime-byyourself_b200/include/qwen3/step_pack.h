// qwen3/step_pack.h - the integer metadata of one step, packed into ONE buffer that goes to the device
// with one copy: token ids, the sequence and the position of every token, the slots, starts and first
// positions of the sequences, the rows whose logits are wanted, and the page rows of the step's
// sequences for every layer group.  Kernels read these sections through the offsets of `StepLayout`.
//
// The reference passes a rectangular [B, S] batch with one shared start position
// (src/model/model.cpp:107-147); here a step is a packed list of sequences of unequal length, each with
// its own position (its slot's length in the cache book).
//
// Header-only C++17.
#pragma once

#include <cstdint>
#include <vector>

#include "cache_book.h"

namespace qwen3 {

// Offsets (in int32 elements) of the sections of a step's metadata buffer; every section starts at a
// multiple of four elements.
struct StepLayout {
    int token_ids = 0, token_seq = 0, token_pos = 0, seq_slots = 0, seq_start = 0, seq_pos0 = 0, want_rows = 0, total = 0;
    std::vector<int> tables;        // one [n_seqs, pages_per_slot] section per layer group

    StepLayout() = default;
    StepLayout(int n_tokens, int n_seqs, int n_want, int n_groups, int pages_per_slot) {
        auto align4 = [](int n) { return (n + 3) & ~3; };
        int o = 0;
        token_ids = o; o += align4(n_tokens);
        token_seq = o; o += align4(n_tokens);
        token_pos = o; o += align4(n_tokens);
        seq_slots = o; o += align4(n_seqs);
        seq_start = o; o += align4(n_seqs + 1);
        seq_pos0 = o; o += align4(n_seqs);
        want_rows = o; o += align4(n_want > 1 ? n_want : 1);
        for (int g = 0; g < n_groups; ++g) {
            tables.push_back(o);
            o += align4(n_seqs * pages_per_slot);
        }
        total = o;
    }
};

// A step of `n_seqs` sequences: sequence i brings n_new[i] tokens (its ids follow those of sequence i - 1 in
// `token_ids`) to slot slots[i], whose length in `book` is the position of its first token.  `book.reserve`
// must have made room already: the page rows are read here.  `out` holds layout.total elements.
inline void pack_step(const CacheBook& book, const StepLayout& lay, const int* slots, const int64_t* n_new, int n_seqs,
                      const int32_t* token_ids, const int32_t* want_rows, int n_want, int32_t* out) {
    int64_t t = 0;
    for (int i = 0; i < n_seqs; ++i) {
        const int64_t pos0 = book.length(slots[i]);
        out[lay.seq_slots + i] = slots[i];
        out[lay.seq_start + i] = (int32_t)t;
        out[lay.seq_pos0 + i] = (int32_t)pos0;
        for (int64_t k = 0; k < n_new[i]; ++k, ++t) {
            out[lay.token_ids + t] = token_ids ? token_ids[t] : 0;
            out[lay.token_seq + t] = i;
            out[lay.token_pos + t] = (int32_t)(pos0 + k);
        }
    }
    out[lay.seq_start + n_seqs] = (int32_t)t;
    for (int r = 0; r < n_want; ++r) out[lay.want_rows + r] = want_rows[r];
    const int P = book.pages_per_slot();
    for (int g = 0; g < book.n_groups(); ++g)
        for (int i = 0; i < n_seqs; ++i) {
            const int32_t* row = book.group(g).row(slots[i]);
            for (int p = 0; p < P; ++p) out[lay.tables[g] + i * P + p] = row[p];
        }
}

// A decode step of a fixed number of `rows`, of which the first `n_live` belong to sequences (one token
// each) and the rest are padding: token 0 at position 0 of the spare slot (number n_slots) and the spare
// page (number n_pages), which belong to no sequence.  Every row's logits are wanted.
inline void pack_decode_step(const CacheBook& book, const StepLayout& lay, int rows, const int* slots, int n_live,
                             const int32_t* token_ids, int32_t* out) {
    const int P = book.pages_per_slot();
    for (int i = 0; i < rows; ++i) {
        const bool live = i < n_live;
        const int32_t pos = live ? (int32_t)book.length(slots[i]) : 0;
        out[lay.token_ids + i] = live && token_ids ? token_ids[i] : 0;
        out[lay.token_seq + i] = i;
        out[lay.token_pos + i] = pos;
        out[lay.seq_slots + i] = live ? slots[i] : book.n_slots();
        out[lay.seq_start + i] = i;
        out[lay.seq_pos0 + i] = pos;
        out[lay.want_rows + i] = i;
    }
    out[lay.seq_start + rows] = rows;
    for (int g = 0; g < book.n_groups(); ++g)
        for (int i = 0; i < rows; ++i) {
            int32_t* to = out + lay.tables[g] + i * P;
            if (i < n_live) {
                const int32_t* row = book.group(g).row(slots[i]);
                for (int p = 0; p < P; ++p) to[p] = row[p];
            } else {
                for (int p = 0; p < P; ++p) to[p] = book.n_pages();
            }
        }
}

}  // namespace qwen3
