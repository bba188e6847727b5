"""The cache's bookkeeping (no GPU): no slot or page lost, held twice or freed twice."""

import random

import pytest
import torch

from dryft_flash_infer_b200.cache import CacheError, FreeList, GroupPages, SequenceCache, SlotBook
from dryft_flash_infer_b200.parts import KVNeed, StateNeed


def test_free_list_hands_out_each_id_once_and_takes_it_back_once():
    ids = FreeList(3, what="slot")
    got = [ids.take(), ids.take(), ids.take()]
    assert sorted(got) == [0, 1, 2]
    with pytest.raises(CacheError, match="out of slots"):
        ids.take()
    ids.give_back(1)
    with pytest.raises(CacheError, match="already free"):
        ids.give_back(1)
    with pytest.raises(CacheError, match="never handed out"):
        ids.give_back(17)
    assert ids.take() == 1  # a freed id is used again
    ids.check()


def test_pages_grow_with_the_sequence_and_come_back():
    pages = GroupPages(n_pages=5, page_size=64, name="g")   # page 0 is never handed out
    book = SlotBook(2, [pages], max_context=256)
    a = book.open()
    book.reserve(a, 65)
    book.advance(a, 65)
    assert len(pages.pages_of[a]) == 2 and 0 not in pages.pages_of[a]
    book.reserve(a, 1)          # 66 tokens still fit two pages
    assert len(pages.pages_of[a]) == 2
    b = book.open()
    book.reserve(b, 128)
    with pytest.raises(CacheError, match="out of cache pages"):
        book.reserve(a, 100)    # would need a third page, none is free
    with pytest.raises(CacheError, match="max_context"):
        book.reserve(b, 300)
    book.check()
    book.close(a)
    with pytest.raises(CacheError, match="freed twice"):
        book.close(a)
    book.reserve(b, 256)        # the freed pages are used again
    book.check()
    book.close(b)
    assert pages.pool.free == 4 and book.slots.free == 2
    book.check()


def test_window_group_takes_its_ring_at_once():
    ring = GroupPages(n_pages=1 + 2 * 3, page_size=64, ring_tokens=192, name="ring")
    book = SlotBook(3, [ring], max_context=100000)
    a, b = book.open(), book.open()
    assert len(ring.pages_of[a]) == 3 and len(ring.pages_of[b]) == 3
    book.reserve(a, 5000)       # a ring never grows
    assert len(ring.pages_of[a]) == 3
    with pytest.raises(CacheError):
        book.open()             # a third ring does not fit: the slot is not lost either
    book.check()
    assert book.slots.free == 1
    book.close(a)
    c = book.open()
    assert c == a
    book.check()


def test_random_open_close_keeps_the_books_straight():
    rng = random.Random(0)
    full = GroupPages(n_pages=1 + 40, page_size=64, name="full")
    ring = GroupPages(n_pages=1 + 6 * 2, page_size=64, ring_tokens=128, name="ring")
    book = SlotBook(6, [full, ring], max_context=1024)
    live = []
    for _ in range(2000):
        action = rng.random()
        try:
            if action < 0.3 and len(live) < 6:
                live.append(book.open())
            elif action < 0.5 and live:
                book.close(live.pop(rng.randrange(len(live))))
            elif live:
                slot = rng.choice(live)
                n = rng.randint(1, 200)
                book.reserve(slot, n)
                book.advance(slot, n)
        except CacheError:
            pass
        book.check()
    for slot in live:
        book.close(slot)
    book.check()
    assert full.pool.free == 40 and ring.pool.free == 12 and book.slots.free == 6


def test_groups_by_need_and_state_area():
    needs = {0: KVNeed(2, 16), 1: KVNeed(2, 16, window=100), 2: KVNeed(2, 16), 3: KVNeed(2, 16, window=100),
             4: KVNeed(4, 32)}
    cache = SequenceCache(needs, {1: StateNeed((3, 5))}, max_tokens=640, max_seqs=4, max_context=640,
                          step_tokens=64, dtype=torch.float32, device="cpu")
    assert len(cache.groups) == 3
    by_ids = {tuple(g.cache_ids): g for g in cache.groups}
    assert by_ids[(0, 2)].k.shape == (2, 11, 2, 64, 16) and by_ids[(0, 2)].ring_tokens == 0
    assert by_ids[(1, 3)].ring_tokens == 192            # window 100 + a pass of 64 - 1, in pages of 64
    assert by_ids[(1, 3)].k.shape == (2, 1 + 4 * 3, 2, 64, 16)
    assert by_ids[(4,)].k.shape == (1, 11, 4, 64, 32)
    a = cache.open_slot()
    cache.state[1][a] += 1.0
    cache.close_slot(a)
    again = cache.open_slot()
    assert again == a and float(cache.state[1][again].abs().sum()) == 0.0  # state starts at zero for the next holder
    cache.book.reserve(again, 100)
    import numpy as np
    table = np.full((1, 4), -1, dtype=np.int32)
    cache.fill_block_table(table, [again], cache.group_of[0][0], 4)
    assert (table[0, :2] > 0).all() and (table[0, 2:] == 0).all()
    view = cache.layer_view(2, [torch.zeros(1, 4, dtype=torch.int32)] * 3, True)
    assert view.k.data_ptr() == by_ids[(0, 2)].k[1].data_ptr() and view.ring_tokens == 0


def test_a_step_laid_out_at_a_larger_shape_keeps_its_spare_rows_away_from_live_pages():
    """The layout that lets short prompt steps share buffers: rows past the step's own belong to no
    sequence and point at the null page; the step's own numbers are where they are without padding."""
    from dryft_flash_infer_b200.engine import StepContext, StepEntry
    from dryft_flash_infer_b200.engine.prefill import shape_for

    cache = SequenceCache({0: KVNeed(2, 16)}, {}, max_tokens=640, max_seqs=4, max_context=320, step_tokens=64,
                          dtype=torch.float32, device="cpu")
    a, b = cache.open_slot(), cache.open_slot()
    cache.book.reserve(a, 70)
    cache.book.advance(a, 70)           # a has 70 tokens already: its share of the step starts there
    entries = [StepEntry(a, [5, 6, 7], [2]), StepEntry(b, list(range(1, 101)), [0, 99])]
    for e in entries:
        cache.book.reserve(e.slot, len(e.tokens))
    assert shape_for(entries) == (128, 4, 4)
    assert shape_for([StepEntry(a, [1], [0]), StepEntry(b, [2], [0])]) is None            # a decode step
    assert shape_for([StepEntry(a, list(range(2000)), [0])]) is None                     # too long
    assert shape_for([StepEntry(a, [1, 2], [])]) is None                                 # nothing wanted
    plain = StepContext(entries, cache, "cpu")
    buffer = torch.full((4096,), -7, dtype=torch.int32)
    padded = StepContext(entries, cache, "cpu", table_widths=[5], shape=(128, 4, 4), into=buffer)
    assert (padded.n_rows, padded.n_seqs, padded.n_wanted) == (128, 4, 4)
    assert (padded.own_rows, padded.own_seqs, padded.own_wanted) == (103, 2, 3)
    assert not padded.all_decode and not padded.wants_every_row and padded.max_q_len == 128
    assert torch.equal(padded.tokens[:103], plain.tokens) and (padded.tokens[103:] == 0).all()
    assert torch.equal(padded.row_pos[:103], plain.row_pos) and (padded.row_pos[103:] == 0).all()
    assert torch.equal(padded.row_seq[:103], plain.row_seq) and (padded.row_seq[103:] == 3).all()
    assert padded.cu_rows.tolist() == [0, 3, 103, 103, 103]
    assert padded.seq_start.tolist() == [70, 0, 0, 0] and padded.seq_qlen.tolist() == [3, 100, 0, 0]
    assert padded.wanted_rows.tolist() == [2, 3, 102, 0]
    table = padded.block_tables[0]
    assert table.shape == (4, 5) and (table[2:] == 0).all()                # the spare sequences: the null page only
    assert torch.equal(table[:2, :2], plain.block_tables[0][:, :2]) and (table[:2, :2] > 0).all()
    assert padded.block_tables[0].data_ptr() >= buffer.data_ptr()          # it lives in the buffer it was given
    with pytest.raises(ValueError, match="does not fit the shape"):
        StepContext(entries, cache, "cpu", table_widths=[5], shape=(128, 2, 4), into=buffer)   # no sequence to spare
