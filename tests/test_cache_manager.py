"""The cache manager on the host: no page lost, held twice or freed twice; windows; reuse (no GPU)."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from lite_lang_b200.cache import CacheError, CacheManager, PageAllocator, PagedGroupSpec, StateGroupSpec


def mgr(num_pages=8, page_size=4, max_requests=4, max_len=64, window=None, extra_window=None):
    groups = [PagedGroupSpec(2, 16, window, 2)]
    pages = [num_pages]
    if extra_window is not None:
        groups.append(PagedGroupSpec(2, 16, extra_window, 1))
        pages.append(num_pages)
    groups.append(StateGroupSpec((3,), "float32", 1))
    return CacheManager(groups, pages, page_size, max_requests, max_len)


def test_allocator_is_lifo_and_refuses_double_free():
    a = PageAllocator(4)
    p = a.alloc(3)
    assert p == [0, 1, 2] and a.num_free == 1
    a.free([1])
    assert a.alloc(1) == [1]                      # the page given back is handed out next
    assert a.alloc(5) is None and a.num_free == 1  # refusal changes nothing
    a.free([0])
    with pytest.raises(CacheError):
        a.free([0])
    with pytest.raises(CacheError):
        a.free([3])                               # never handed out


def test_reserve_advance_close():
    m = mgr()
    s = m.open()
    assert m.reserve(s, 5)                         # 2 pages of 4
    assert m.pages_of(0, s) == [0, 1] and m.num_free_pages() == 6
    assert m.reserve(s, 8) and m.num_free_pages() == 6    # still inside the pages held
    m.advance(s, 5)
    assert m.length(s) == 5
    assert m.slot_of_position(0, s, 4) == 1 * 4 + 0
    assert (m.block_tables[0][s, :2] == [0, 1]).all() and m.block_tables[0][s, 2] == -1
    m.check_invariants()
    m.close(s)
    assert m.num_free_pages() == 8 and (m.block_tables[0] == -1).all()
    m.check_invariants()
    with pytest.raises(CacheError):
        m.close(s)


def test_running_out_is_an_answer_not_an_exception():
    m = mgr(num_pages=3)
    a, b = m.open(), m.open()
    assert m.reserve(a, 8)
    assert not m.can_reserve(b, 8)
    assert not m.reserve(b, 8) and m.pages_of(0, b) == []     # all or nothing
    assert m.reserve(b, 4)
    assert m.num_free_pages() == 0
    assert not m.reserve(a, 9)
    m.check_invariants()
    assert not m.reserve(a, 65)                               # beyond max_model_len


def test_slots_run_out_and_come_back():
    m = mgr(max_requests=2)
    a, b = m.open(), m.open()
    assert m.open() is None
    m.close(a)
    assert m.open() == a
    assert m.take_opened_slots() == [a, b, a]
    assert m.take_opened_slots() == []


def test_pages_are_used_again():
    m = mgr(num_pages=4)
    a = m.open()
    m.reserve(a, 16)
    first = m.pages_of(0, a)
    m.advance(a, 16)
    m.close(a)
    b = m.open()
    m.reserve(b, 8)
    assert set(m.pages_of(0, b)) <= set(first)
    assert m.pages_reused == 2


def test_window_gives_pages_back_as_it_moves():
    m = mgr(num_pages=6, window=6)
    s = m.open()
    assert m.reserve(s, 10)
    m.advance(s, 10)       # next token at 10 reads positions 5..10 -> page 0 (0..3) is passed
    assert m.pages_of(0, s) == [-1, 1, 2]
    assert m.block_tables[0][s, 0] == -1 and m.num_free_pages(0) == 4
    with pytest.raises(CacheError):
        m.slot_of_position(0, s, 2)
    assert m.reserve(s, 14)                 # the page given back is taken again at once
    assert m.pages_of(0, s)[3] == 0
    m.advance(s, 14)       # reads 9..14 -> pages 0 and 1 (positions < 8) passed
    assert m.pages_of(0, s)[:2] == [-1, -1]
    m.check_invariants()
    m.close(s)
    assert m.num_free_pages(0) == 6
    m.check_invariants()


def test_groups_have_pages_of_their_own():
    m = mgr(num_pages=5, extra_window=4)
    s = m.open()
    assert m.reserve(s, 12)
    m.advance(s, 12)
    assert m.num_free_pages(0) == 2          # full attention keeps its 3 pages
    assert m.num_free_pages(1) == 4          # the windowed group kept the page of positions 8..11 only
    assert m.pages_of(1, s)[:2] == [-1, -1]
    assert m.num_free_pages() == 2           # the scarcest group decides
    m.check_invariants()


def test_dirty_rows_are_reported_once():
    m = mgr()
    a = m.open()
    m.reserve(a, 3)
    assert m.take_dirty_rows(0) == [a]
    assert m.take_dirty_rows(0) == []
    m.reserve(a, 4)
    assert m.take_dirty_rows(0) == []        # no new page, nothing to push
    m.reserve(a, 5)
    assert m.take_dirty_rows(0) == [a]


def test_advance_without_pages_is_a_bug():
    m = mgr()
    s = m.open()
    m.reserve(s, 4)
    with pytest.raises(CacheError):
        m.advance(s, 5)


@settings(max_examples=60, deadline=None)
@given(seed=st.integers(0, 10 ** 6), num_pages=st.integers(2, 12), window=st.sampled_from([None, 3, 7, 16]))
def test_random_orders_keep_the_invariants(seed, num_pages, window):
    rng = random.Random(seed)
    m = mgr(num_pages=num_pages, page_size=4, max_requests=4, max_len=40, window=window, extra_window=5)
    live = {}
    for _ in range(120):
        op = rng.random()
        if op < 0.25 and m.num_free_slots:
            s = m.open()
            live[s] = 0
        elif op < 0.85 and live:
            s = rng.choice(list(live))
            add = rng.randint(1, 9)
            if m.reserve(s, live[s] + add):
                live[s] += add
                m.advance(s, live[s])
            else:
                assert live[s] + add > 40 or not m.can_reserve(s, live[s] + add)
        elif live:
            s = rng.choice(list(live))
            m.close(s)
            del live[s]
        m.check_invariants()
    for s in list(live):
        m.close(s)
    m.check_invariants()
    assert m.num_free_pages(0) == num_pages and m.num_free_pages(1) == num_pages
    assert m.num_free_slots == 4


def test_groups_may_have_different_page_counts_and_every_group_is_asked():
    """A group with a window needs few pages; the most a request may grow to is what every group can take."""
    groups = [PagedGroupSpec(2, 16, None, 2), PagedGroupSpec(2, 16, 8, 1)]
    m = CacheManager(groups, [10, 4], 4, 4, 64)
    assert m.capacity_tokens() == 40                    # the group that keeps every position sets it
    s = m.open()
    assert m.max_reservable(s) == 16                    # the windowed group has 4 pages
    assert not m.reserve(s, 17) and m.reserve(s, 16)
    m.advance(s, 16)                                    # the window is 8: pages of positions < 9 go back
    assert m.pages_of(1, s)[:2] == [-1, -1] and m.num_free_pages(1) == 2
    assert m.max_reservable(s) == 24                    # 4 logical pages so far + 2 free
    assert m.reserve(s, 24)
    m.advance(s, 24)
    assert m.max_reservable(s) == 32
    # a request of 40 tokens fits alone (in steps of 4 tokens the windowed group needs 4 pages), one of 41 does not
    assert m.can_ever_hold(40, step_tokens=4) and not m.can_ever_hold(44, step_tokens=4)
    assert not m.can_ever_hold(40, step_tokens=12)      # 8 + 12 tokens of window and step need 6 pages
    m.check_invariants()
    only_windows = CacheManager([PagedGroupSpec(1, 8, 8, 1)], [9], 4, 4, 64)
    assert only_windows.capacity_tokens() == (9 // 4) * 64     # requests whose windows fit, times the longest


def test_pages_are_shared_out_from_a_budget_of_bytes():
    from lite_lang_b200.cache.sizing import page_bytes, plan_pages, state_bytes
    full = PagedGroupSpec(2, 16, None, 3)                      # keys and values 16 wide, 3 planes
    narrow = PagedGroupSpec(2, 16, None, 1, value_head_dim=8)  # values half as wide as the keys
    latent = PagedGroupSpec(1, 24, None, 1, value_head_dim=0)  # one vector a token, no value plane
    windowed = PagedGroupSpec(2, 16, 8, 2)
    state = StateGroupSpec((5, 3), "float32", 2)
    assert page_bytes(full, 4, 2) == 3 * 2 * 4 * 32 * 2
    assert page_bytes(narrow, 4, 2) == 2 * 4 * 24 * 2 and page_bytes(latent, 4, 2) == 1 * 4 * 24 * 2
    assert state_bytes(state, 4, 2) == 2 * 4 * 15 * 4
    # without a window every group gets the same number of pages, and the state records come off the budget
    budget = 100 * (page_bytes(full, 4, 2) + page_bytes(narrow, 4, 2)) + state_bytes(state, 4, 2) + 7
    assert plan_pages([full, state, narrow], budget, 4, 2, 4, 10 ** 6, 8) == [100, 100]
    # a windowed group stops at what its request slots can ever use; the others get what that leaves
    cap = 4 * windowed.pages_a_request_needs(10 ** 6, 4, 8)    # 4 slots x (ceil((8 + 8) / 4) + 1) pages
    assert cap == 20
    budget = 100 * page_bytes(full, 4, 2) + cap * page_bytes(windowed, 4, 2)
    assert plan_pages([full, windowed], budget, 4, 2, 4, 10 ** 6, 8) == [100, 20]
    # nobody gets more than every slot at full length needs; never fewer than one page
    assert plan_pages([full], 10 ** 12, 4, 2, 4, 40, 8) == [40]
    assert plan_pages([full, windowed], 10, 4, 2, 4, 40, 8) == [1, 1]
