"""The cache's bookkeeping: no slot or page is lost, held twice or freed twice; lengths per
sequence; groups with storage of their own; window groups return dead pages; state layers."""
import numpy as np
import pytest

from qwen3_b200.cache import PAGE_TOKENS, CacheBook, CacheError, CacheFull, CacheNeed

FULL = CacheNeed("full", 2, 16)


def test_each_slot_is_handed_out_once_and_taken_back_once():
    book = CacheBook([FULL], max_tokens=8 * PAGE_TOKENS, max_seq_len=PAGE_TOKENS, n_slots=3)
    got = [book.alloc_slot(), book.alloc_slot(), book.alloc_slot()]
    assert sorted(got) == [0, 1, 2] and book.slots.n_free == 0
    with pytest.raises(CacheFull):
        book.alloc_slot()
    book.free_slot(got[1])
    with pytest.raises(CacheError):
        book.free_slot(got[1])               # freed twice
    with pytest.raises(CacheError):
        book.free_slot(7)                    # never handed out
    assert not book.slots.is_held(got[1]) and book.slots.is_held(got[0])
    assert book.alloc_slot() == got[1] and book.slots.held == frozenset(got)


def test_lengths_pages_and_reuse():
    book = CacheBook([FULL, FULL, FULL], max_tokens=5 * PAGE_TOKENS, max_seq_len=4 * PAGE_TOKENS)
    assert book.n_pages == 5 and book.pages_per_slot == 4 and len(book.groups) == 1 and book.groups[0].layers == [0, 1, 2]
    a, b = book.alloc_slot(), book.alloc_slot()
    book.reserve([(a, 70), (b, 1)])
    book.commit([(a, 70), (b, 1)])
    assert (book.length(a), book.length(b)) == (70, 1) and book.pages_held() == 3
    pages_a, pages_b = book.groups[0].held_pages(a), book.groups[0].held_pages(b)
    assert len(pages_a) == 2 and len(pages_b) == 1 and not set(pages_a) & set(pages_b)
    for _ in range(58):                       # a grows to 128: still two pages
        book.reserve([(a, 1), (b, 1)])
        book.commit([(a, 1), (b, 1)])
    assert book.length(a) == 128 and book.groups[0].held_pages(a) == pages_a and book.pages_held() == 3
    book.reserve([(a, 1)])                    # position 128 opens a third page
    book.commit([(a, 1)])
    assert len(book.groups[0].held_pages(a)) == 3
    rows = book.page_rows(0, [b, a])
    assert rows.shape == (2, 4) and list(rows[1][:3]) == book.groups[0].held_pages(a) and rows[0][1] == -1
    book.free_slot(a)
    assert book.pages_held() == 1 and book.length(a) == 0
    with pytest.raises(CacheError):
        book.free_slot(a)
    c = book.alloc_slot()
    assert c == a and book.length(c) == 0 and book.groups[0].held_pages(c) == []
    book.reserve([(c, 200)])
    assert set(book.groups[0].held_pages(c)) & set(pages_a)      # pages are used again


def test_a_step_that_does_not_fit_changes_nothing():
    book = CacheBook([FULL], max_tokens=3 * PAGE_TOKENS, max_seq_len=2 * PAGE_TOKENS)
    a, b = book.alloc_slot(), book.alloc_slot()
    book.reserve([(a, 64)])
    book.commit([(a, 64)])
    before = book.groups[0].table.copy()
    with pytest.raises(CacheFull):
        book.reserve([(a, 10), (b, 100)])     # 1 + 2 pages wanted, 2 free
    with pytest.raises(CacheFull):
        book.reserve([(a, 65)])               # beyond the sequence capacity
    with pytest.raises(CacheError):
        book.reserve([(a, 1), (a, 1)])
    with pytest.raises(CacheError):
        book.reserve([(5, 1)])
    with pytest.raises(CacheError):
        book.reserve([(a, 0)])
    assert np.array_equal(before, book.groups[0].table) and book.groups[0].n_free == 2


def test_a_cancelled_step_gives_its_pages_back_and_can_be_tried_again():
    window = CacheNeed("window", 1, 16, window=70)
    book = CacheBook([FULL, window], max_tokens=6 * PAGE_TOKENS, max_seq_len=5 * PAGE_TOKENS)
    a, b = book.alloc_slot(), book.alloc_slot()
    book.reserve([(a, 100), (b, 3)])
    book.commit([(a, 100), (b, 3)])
    tables = [g.table.copy() for g in book.groups]
    free = [sorted(g._free) for g in book.groups]
    step = [(a, 130), (b, 62)]                  # two more pages for a (three in the window group's count too), one for b
    book.reserve(step)
    assert all(g.n_free < len(f) for g, f in zip(book.groups, free))
    book.cancel(step)
    assert book.length(a) == 100 and book.length(b) == 3
    for g, t, f in zip(book.groups, tables, free):
        assert np.array_equal(g.table, t) and sorted(g._free) == f
    book.reserve(step)                          # the same step again: nothing was lost, so it still fits
    book.commit(step)
    assert book.length(a) == 230 and book.length(b) == 65
    book.free_slot(a); book.free_slot(b)
    assert all(g.n_free == g.n_pages for g in book.groups)


def test_random_schedule_never_loses_or_doubles_a_page():
    rng = np.random.default_rng(0)
    book = CacheBook([FULL, FULL], max_tokens=40 * PAGE_TOKENS, max_seq_len=9 * PAGE_TOKENS, n_slots=8)
    live = {}
    for _ in range(3000):
        action = rng.integers(0, 10)
        if action < 2 and len(live) < 8:
            live[book.alloc_slot()] = 0
        elif action < 3 and live:
            slot = list(live)[rng.integers(len(live))]
            book.free_slot(slot)
            del live[slot]
        elif live:
            step = [(s, int(rng.integers(1, 100))) for s in live if rng.random() < 0.6]
            if not step:
                continue
            try:
                book.reserve(step)
            except CacheFull:
                continue
            if rng.random() < 0.15:             # the step's launch failed: what was reserved goes back
                book.cancel(step)
                continue
            book.commit(step)
            for s, n in step:
                live[s] += n
        held = [p for s in live for p in book.groups[0].held_pages(s)]
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) + book.groups[0].n_free == book.n_pages, "a page is lost"
        assert sorted(set(held) | set(book.groups[0]._free)) == list(range(book.n_pages))
        for s, n in live.items():
            assert book.length(s) == n and len(book.groups[0].held_pages(s)) == -(-n // PAGE_TOKENS)
        assert book.slots.held == frozenset(live) and book.slots.n_free == 8 - len(live)
    for s in list(live):
        book.free_slot(s)
    assert book.groups[0].n_free == book.n_pages and book.slots.n_free == 8


def test_groups_with_different_needs_have_storage_of_their_own():
    window = CacheNeed("window", 1, 32, window=100)
    state_only = CacheNeed("none", state_shape=(4, 8))
    both = CacheNeed("full", 2, 16, state_shape=(3,))
    book = CacheBook([FULL, window, None, state_only, both, window], max_tokens=20 * PAGE_TOKENS,
                     max_seq_len=20 * PAGE_TOKENS)
    assert [g.layers for g in book.groups] == [[0, 4], [1, 5]]
    assert book.group_of_layer == {0: 0, 4: 0, 1: 1, 5: 1}
    assert book.state_layers == {3: (4, 8), 4: (3,)}
    s = book.alloc_slot()
    book.reserve([(s, 400)])
    book.commit([(s, 400)])
    full, win = book.groups
    assert len(full.held_pages(s)) == 7
    # a query at position >= 400 reads keys > 300: pages 0..3 (positions < 256) are dead, page 4 (256..319) is not
    assert len(win.held_pages(s)) == 3 and list(win.table[s][:5]) == [-1, -1, -1, -1, win.table[s][4]]
    for _ in range(200):
        book.reserve([(s, 1)])
        book.commit([(s, 1)])
    assert len(full.held_pages(s)) == 10 and len(win.held_pages(s)) <= 3
    book.free_slot(s)
    assert full.n_free == 20 and win.n_free == 20


def test_cache_need_checks():
    with pytest.raises(ValueError):
        CacheNeed("ring", 1, 16)
    with pytest.raises(ValueError):
        CacheNeed("window", 1, 16)
    with pytest.raises(ValueError):
        CacheNeed("full", 0, 16)


def test_guarded_scratch_names_the_buffer_that_was_written_beyond():
    """The guard zones around activation buffers (a debugging mode of the engine's scratch): a write one
    element behind or before a buffer is found and named; buffers of other names and sizes are not."""
    torch = pytest.importorskip("torch")
    from qwen3_b200.engine.context import Scratch
    scratch = Scratch("cpu", guard=True)
    a = scratch.get("a", (3, 5), torch.float32)
    b = scratch.get("b", (7,), torch.bfloat16)
    assert a.shape == (3, 5) and b.shape == (7,) and scratch.get("a", (3, 5), torch.float32).data_ptr() == a.data_ptr()
    assert scratch.get("a", (4, 5), torch.float32).data_ptr() != a.data_ptr()        # another size: a buffer of its own
    a.fill_(1.0)
    b.fill_(2.0)
    assert scratch.violations() == []
    beyond = torch.as_strided(b, (8,), (1,))                   # one element past the end
    beyond[7] = 3.0
    assert scratch.violations() == [("b", torch.bfloat16, 7)]
    before = torch.as_strided(a, (1,), (1,), storage_offset=a.storage_offset() - 1)
    before[0] = 0.0
    assert sorted(v[0] for v in scratch.violations()) == ["a", "b"]
    plain = Scratch("cpu")
    assert plain.get("x", (4,), torch.float32).numel() == 4 and plain.violations() == []
