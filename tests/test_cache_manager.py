"""The cache manager (host, C++): no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; slots; all-or-nothing reservation (no GPU)."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from llmengine.cache import host_module

H = host_module()


def make(page=4, pages=(16,), windows=(0,), slots=4):
    return H.CacheManager(page, [H.GroupSpec(p, w) for p, w in zip(pages, windows)], slots)


def test_pages_fifo_and_tables():
    cm = make()
    assert cm.add_request(10) == 0 and cm.add_request(11) == 1
    assert cm.reserve(10, 5) and cm.block_table(10) == [0, 1]
    assert cm.reserve(11, 1) and cm.block_table(11) == [2]
    cm.advance(10, 5)
    assert cm.length(10) == 5 and cm.reserve(10, 3) and cm.block_table(10) == [0, 1]  # 8 tokens fit 2 pages
    assert cm.reserve(10, 4) and cm.block_table(10) == [0, 1, 3]
    cm.check()
    cm.release(10)
    assert cm.free_pages() == 15 and cm.free_slots == 3
    # freed pages go to the back of the list: they are used again after the untouched ones
    cm.add_request(12)
    assert cm.reserve(12, 4 * 13) and cm.block_table(12)[-3:] == [14, 15, 0]
    cm.check()


def test_reserve_is_all_or_nothing_across_groups():
    cm = make(pages=(8, 2), windows=(0, 0))
    cm.add_request(1)
    assert not cm.reserve(1, 12)  # needs 3 pages in each group; the second has 2
    assert cm.free_pages(0) == 8 and cm.free_pages(1) == 2 and cm.block_table(1, 0) == []
    assert cm.reserve(1, 8)
    cm.check()


def test_window_group_gives_pages_back_once_passed():
    cm = make(page=4, pages=(32, 6), windows=(0, 6))
    cm.add_request(1)
    assert cm.reserve(1, 10)
    cm.advance(1, 10)  # next query is position 10: it reads keys 5..10, page 0 (0..3) is dead
    assert cm.block_table(1, 1) == [-1, 1, 2] and cm.free_pages(1) == 4
    assert cm.block_table(1, 0) == [0, 1, 2]
    for _ in range(40):  # a long request lives on a handful of window pages
        assert cm.reserve(1, 1)
        cm.advance(1, 1)
        cm.check()
    assert cm.length(1) == 50 and sum(p >= 0 for p in cm.block_table(1, 1)) <= 3
    assert sum(p >= 0 for p in cm.block_table(1, 0)) == 13
    cm.release(1)
    assert cm.free_pages(0) == 32 and cm.free_pages(1) == 6
    cm.check()


def test_slots_run_out_and_come_back():
    cm = make(slots=2)
    assert cm.add_request(1) == 0 and cm.add_request(2) == 1 and cm.add_request(3) == -1
    assert not cm.has_request(3)
    cm.release(1)
    assert cm.add_request(3) == 0
    cm.check()


def test_misuse_is_refused():
    cm = make()
    cm.add_request(1)
    with pytest.raises(ValueError, match="already exists"):
        cm.add_request(1)
    with pytest.raises(IndexError):
        cm.release(2)
    cm.reserve(1, 3)
    with pytest.raises(RuntimeError, match="past its reserved"):
        cm.advance(1, 5)
    cm.release(1)
    with pytest.raises(IndexError):  # freed twice
        cm.release(1)
    with pytest.raises(ValueError):
        make(page=0)
    cm.check()


@settings(max_examples=60, deadline=None)
@given(seed=st.integers(0, 10 ** 6), page=st.sampled_from([1, 4, 16]), window=st.sampled_from([0, 5, 33]))
def test_random_orders_keep_every_page_accounted_for(seed, page, window):
    rng = random.Random(seed)
    pages = rng.randint(4, 40)
    cm = make(page=page, pages=(pages, pages), windows=(0, window), slots=5)
    live, next_id = {}, 0
    for _ in range(200):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            assert cm.add_request(next_id) >= 0
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 30])
            free_before = (cm.free_pages(0), cm.free_pages(1))
            if cm.reserve(rid, n):
                cm.advance(rid, n)
                live[rid] += n
                assert cm.length(rid) == live[rid]
                # every position a later query can read is backed by a page
                for g, w in ((0, 0), (1, window)):
                    t = cm.block_table(rid, g)
                    lo = max(0, live[rid] - w + 1) if w else 0
                    assert all(t[p // page] >= 0 for p in range(lo, live[rid]))
            else:
                assert (cm.free_pages(0), cm.free_pages(1)) == free_before  # nothing taken on failure
        elif live:
            rid = rng.choice(list(live))
            cm.release(rid)
            del live[rid]
        cm.check()
        held = [p for rid in live for p in cm.block_table(rid, 0) if p >= 0]
        assert len(held) == len(set(held)) and len(held) + cm.free_pages(0) == pages
    for rid in list(live):
        cm.release(rid)
    cm.check()
    assert cm.free_pages(0) == pages and cm.free_pages(1) == pages and cm.free_slots == 5


def test_step_batch_builder_lays_out_a_mixed_batch():
    import numpy as np
    cm = make(page=4, pages=(16,), windows=(0,))
    cm.add_request(5); cm.add_request(6)
    cm.reserve(5, 6); cm.advance(5, 6)  # request 5 already holds 6 tokens
    cm.reserve(5, 1); cm.reserve(6, 5)
    e = H.StepEntries()
    e.add(6, [9, 8, 7, 6, 5], [4])
    e.add(5, [3], [0], 0.5, 11, 2)
    assert H.step_caps(cm, e) == (6, 2, 2, 2)
    L = H.StepLayout.make(6, 2, 2, 2, 1)
    buf = np.full(L.total, -7, dtype=np.int32)
    c = H.fill_step(cm, e, L, buf.ctypes.data, False, 256, 128)
    assert (c.n_tokens, c.n_seqs, c.n_rows, c.max_seq_len, c.max_new_tokens, c.decode_only) == (6, 2, 2, 7, 5, False)
    assert buf[L.token_ids:L.token_ids + 6].tolist() == [9, 8, 7, 6, 5, 3]
    assert buf[L.positions:L.positions + 6].tolist() == [0, 1, 2, 3, 4, 6]
    assert buf[L.token_seq:L.token_seq + 6].tolist() == [0, 0, 0, 0, 0, 1]
    assert buf[L.logit_rows:L.logit_rows + 2].tolist() == [4, 5]
    assert buf[L.seq_start:L.seq_start + 2].tolist() == [0, 6] and buf[L.seq_qoff:L.seq_qoff + 3].tolist() == [0, 5, 6]
    assert buf[L.seq_len:L.seq_len + 2].tolist() == [5, 7]
    assert buf[L.block_tables:L.block_tables + 4].tolist() == cm.block_table(6) + cm.block_table(5)
    assert buf[L.row_temperature:L.row_temperature + 2].view(np.float32).tolist() == [0.0, 0.5]
    assert buf[L.row_seed + 1] == 11 and buf[L.row_draw + 1] == 2
    # errors: unknown request, no pages reserved, token out of range, wanted place outside, twice
    for bad, word in ((lambda x: x.add(7, [1], []), "unknown request"), (lambda x: x.add(5, [1, 2], []), "no pages reserved"),
                      (lambda x: x.add(5, [256], []), "out of range"), (lambda x: x.add(5, [1], [1]), "wanted place"),
                      (lambda x: (x.add(5, [1], []), x.add(5, [1], [])), "appears twice"), (lambda x: x.add(5, [], []), "no tokens")):
        e2 = H.StepEntries()
        bad(e2)
        with pytest.raises((ValueError, RuntimeError), match=word):
            H.fill_step(cm, e2, H.StepLayout.make(8, 2, 2, 4, 1), buf.ctypes.data if buf.size >= 64 else 0, False, 256, 128)
    # padded batch (CUDA-graph replays): spare rows point at the null page and the null slot
    e3 = H.StepEntries(); e3.add(5, [3], [0])
    L3 = H.StepLayout.make(4, 4, 4, 3, 1)
    buf3 = np.zeros(L3.total, dtype=np.int32)
    c3 = H.fill_step(cm, e3, L3, buf3.ctypes.data, True, 256, 128)
    assert c3.n_tokens == 1 and c3.decode_only
    assert buf3[L3.block_tables + 3:L3.block_tables + 12].tolist() == [16] * 9
    assert buf3[L3.seq_slot:L3.seq_slot + 4].tolist() == [cm.slot(5), 4, 4, 4]
    assert buf3[L3.positions:L3.positions + 4].tolist() == [6, 0, 0, 0]
