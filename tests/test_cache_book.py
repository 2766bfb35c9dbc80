"""Cache bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from qwen_triton_b200.cache.store import CacheView
from qwen_triton_b200.cache import CacheBook, CacheError, CacheFull, GroupGeometry, SequenceCache
from qwen_triton_b200.parts.base import KVRequest, StateRequest


def make_book(slots=4, pages=8, ring=0):
    return CacheBook(slots, 64, [GroupGeometry(pages), GroupGeometry(pages, ring)] if ring else [GroupGeometry(pages)], 4096)


def test_slots_are_handed_out_given_back_and_used_again():
    book = make_book()
    slots = [book.alloc() for _ in range(4)]
    assert slots == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        book.alloc()
    book.free(2)
    with pytest.raises(CacheError, match="not in use"):
        book.free(2)                                    # freed twice
    assert book.alloc() == 2                            # the slot comes back
    book.check()


def test_pages_follow_the_length_and_return_on_free():
    book = make_book(pages=6)
    a, b = book.alloc(), book.alloc()
    book.extend(a, 1)
    assert len(book.pages(a, 0)) == 1
    book.extend(a, 64)
    assert len(book.pages(a, 0)) == 1
    book.extend(a, 65)
    assert len(book.pages(a, 0)) == 2
    book.extend(b, 200)
    assert len(book.pages(b, 0)) == 4 and book.free_pages(0) == 0
    assert not set(book.pages(a, 0)) & set(book.pages(b, 0))          # no page held twice
    with pytest.raises(CacheFull):
        book.extend(a, 129)
    assert book.length(a) == 65 and len(book.pages(a, 0)) == 2         # a failed extend changes nothing
    assert not book.can_hold({a: 129}) and book.can_hold({a: 128})
    with pytest.raises(CacheError, match="shrink"):
        book.extend(a, 10)
    book.free(b)
    assert book.free_pages(0) == 4
    book.extend(a, 300)
    book.check()


def test_window_group_keeps_a_ring_of_pages():
    book = make_book(pages=16, ring=3)
    slot = book.alloc()
    book.extend(slot, 1000)
    assert len(book.pages(slot, 0)) == 16 and len(book.pages(slot, 1)) == 3
    book.free(slot)
    assert book.free_pages(0) == 16 and book.free_pages(1) == 16
    book.check()


def test_longest_sequence_is_enforced():
    book = CacheBook(2, 64, [GroupGeometry(100)], 128)
    slot = book.alloc()
    with pytest.raises(CacheFull, match="128"):
        book.extend(slot, 129)


def test_random_traffic_keeps_the_books_straight():
    rng = random.Random(7)
    book = make_book(slots=6, pages=40, ring=2)
    live: dict[int, int] = {}
    for _ in range(3000):
        action = rng.random()
        if action < 0.3 and book.free_slot_count():
            slot = book.alloc()
            assert slot not in live
            live[slot] = 0
        elif action < 0.5 and live:
            slot = rng.choice(list(live))
            book.free(slot)
            del live[slot]
        elif live:
            slot = rng.choice(list(live))
            target = live[slot] + rng.randint(1, 300)
            if book.can_hold({slot: target}) and target <= 4096:
                book.extend(slot, target)
                live[slot] = target
            else:
                with pytest.raises(CacheFull):
                    book.extend(slot, target)
        book.check()
        assert book.live_slots() == sorted(live)
        for slot, length in live.items():
            assert book.length(slot) == length
            assert len(book.pages(slot, 0)) == -(-length // 64)
            assert len(book.pages(slot, 1)) == min(-(-length // 64), 2)
    for slot in list(live):
        book.free(slot)
    assert book.free_pages(0) == 40 and book.free_pages(1) == 40 and book.free_slot_count() == 6


def test_groups_by_need_and_shared_entries():
    full, window = KVRequest(2, 16), KVRequest(2, 16, window=24)
    requests = [full, full, window, None, StateRequest((4, 8)), window]
    cache_of = [None, None, None, 1, None, None]
    cache = SequenceCache(requests, cache_of, max_tokens=1000, max_seq_len=512, dtype=None, device=None,
                          chunk_tokens=32, allocate=False)
    assert len(cache.groups) == 2
    assert cache.groups[0].owners == [(0, 0), (1, 0)] and cache.groups[1].owners == [(2, 0), (5, 0)]      # (position, request number)
    assert cache.groups[0].ring_tokens == 0 and cache.groups[1].ring_tokens == 64      # 24 + 32 - 1 rounded up to pages
    assert cache.num_slots == 16 and cache.book.groups[1].ring_pages == 1
    reader = cache.view(3)
    assert reader.group == 0 and not reader.writable                                    # reads the entry of position 1
    assert cache.view(4).group is None and cache.view(2).ring_tokens == 64
    assert cache.max_blocks(0) == 8 and cache.max_blocks(1) == 1


def test_a_layer_with_several_parts_that_keep_something():
    """A position may ask for a list (keys and values beside a fixed-size state): its view is a tuple in that order,
    and a later position that reads its entries sees both, read-only."""
    full = KVRequest(2, 16)
    requests = [full, [full, StateRequest((3,)), None], [None, None, None]]
    cache = SequenceCache(requests, [None, None, 1], max_tokens=256, max_seq_len=128, dtype=None, device=None, allocate=False)
    assert len(cache.groups) == 1 and cache.groups[0].owners == [(0, 0), (1, 0)]
    assert isinstance(cache.view(0), CacheView)
    pair = cache.view(1)
    assert isinstance(pair, tuple) and len(pair) == 3
    assert pair[0].group == 0 and pair[0].writable and pair[1].group is None and pair[2].group is None
    reader = cache.view(2)
    assert len(reader) == 3 and reader[0].group == 0 and not reader[0].writable
