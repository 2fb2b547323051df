"""The cache manager on the host: no page lost, held twice or freed twice."""

import numpy as np
import pytest

from ayaka_py_b200.cache import CacheGroupSpec, CacheManager, NoFreeSlot, OutOfPages
from ayaka_py_b200.parts.base import KVNeed, StateNeed


def manager(pages=9, page_size=4, max_requests=4, max_len=64, window=None, extra=()):
    groups = [CacheGroupSpec("full", KVNeed(2, 16, window), 2), *extra]
    return CacheManager(groups, kv_pages=pages, page_size=page_size, max_requests=max_requests,
                        max_len=max_len, device=None)


def test_reserve_commit_close():
    m = manager()
    a = m.open("a")
    r = m.reserve([(a, 0, 6)])
    assert m.free_pages() == 6 and (m.tables[0][a, :2] > 0).all() and m.tables[0][a, 2] == 0
    m.commit(r)
    assert m.length[a] == 6
    r = m.reserve([(a, 6, 2)])          # fills the second page, no new page
    assert m.free_pages() == 6
    m.commit(r)
    r = m.reserve([(a, 8, 1)])
    assert m.free_pages() == 5
    m.commit(r)
    m.check_invariants()
    m.close(a)
    m.assert_clean()


def test_entry_must_continue_the_request():
    m = manager()
    a = m.open("a")
    with pytest.raises(ValueError):
        m.reserve([(a, 3, 2)])
    m.commit(m.reserve([(a, 0, 3)]))
    with pytest.raises(ValueError):
        m.reserve([(a, 0, 3)])
    with pytest.raises(ValueError):
        m.reserve([(a, 3, 1), (a, 4, 1)])
    with pytest.raises(ValueError):
        m.reserve([(a, 3, 62)])          # beyond max_len
    with pytest.raises(KeyError):
        m.reserve([(3, 0, 1)])


def test_step_is_all_or_nothing():
    m = manager(pages=5)                 # 4 usable pages of 4 tokens
    a, b = m.open("a"), m.open("b")
    with pytest.raises(OutOfPages) as err:
        m.reserve([(a, 0, 9), (b, 0, 8)])       # 3 + 2 pages
    assert err.value.needed == 5 and err.value.free == 4
    assert m.free_pages() == 4 and not m.tables[0].any() and not m.in_step.any()
    r = m.reserve([(a, 0, 9), (b, 0, 4)])
    assert m.free_pages() == 0
    m.rollback(r)
    assert m.free_pages() == 4 and not m.tables[0].any() and m.length[a] == 0
    with pytest.raises(RuntimeError):
        m.commit(r)
    m.check_invariants()


def test_pages_are_used_again():
    m = manager(pages=4)
    a = m.open("a")
    m.commit(m.reserve([(a, 0, 12)]))
    first = set(m.tables[0][a, :3].tolist())
    m.close(a)
    b = m.open("b")
    m.commit(m.reserve([(b, 0, 5)]))
    assert set(m.tables[0][b, :2].tolist()) <= first
    assert m.stats()["groups"]["full"]["reused"] == 2
    m.close(b)
    m.assert_clean()


def test_double_free_and_busy_are_caught():
    m = manager()
    a = m.open("a")
    r = m.reserve([(a, 0, 4)])
    with pytest.raises(RuntimeError):
        m.close(a)                       # inside a step
    with pytest.raises(RuntimeError):
        m.reserve([(a, 0, 4)])
    m.commit(r)
    m.close(a)
    with pytest.raises(KeyError):
        m.close(a)
    with pytest.raises(AssertionError):
        m.pools[0].give(1, 0)            # a free page cannot be freed again


def test_slots_run_out_and_return():
    m = manager(max_requests=2)
    a, b = m.open("a"), m.open("b")
    with pytest.raises(NoFreeSlot):
        m.open("c")
    with pytest.raises(KeyError):
        m.open("a")
    m.close(a)
    assert m.open("c") == a


def test_preempt_keeps_the_slot():
    m = manager()
    a = m.open("a")
    m.commit(m.reserve([(a, 0, 10)]))
    m.preempt(a)
    assert m.length[a] == 0 and m.free_pages() == 8 and "a" in m.slot_of
    m.commit(m.reserve([(a, 0, 3)]))
    m.close(a)
    m.assert_clean()


def test_window_gives_pages_back():
    m = manager(pages=6, page_size=4, window=6)
    a = m.open("a")
    m.commit(m.reserve([(a, 0, 9)]))      # next query at 9 reads keys 4..9: page 0 returns
    assert m.first_page[0][a] == 1 and m.tables[0][a, 0] == 0 and m.free_pages() == 3
    for pos in range(9, 40):              # decodes far beyond the pool's 20 tokens
        m.commit(m.reserve([(a, pos, 1)]))
        m.check_invariants()
        held = int(m.num_pages[0][a] - m.first_page[0][a])
        assert held <= 3
        first_key = max(0, pos + 1 - 6 + 1)
        assert m.first_page[0][a] <= first_key // 4          # a needed key is never given back
    assert m.stats()["groups"]["full"]["reused"] > 0
    m.close(a)
    m.assert_clean()


def test_groups_have_pages_of_their_own_and_state_slots():
    extra = (CacheGroupSpec("win", KVNeed(1, 16, 4), 1), CacheGroupSpec("state", StateNeed((3,)), 2))
    m = manager(pages=6, extra=extra)
    a = m.open("a")
    m.commit(m.reserve([(a, 0, 12)]))
    assert m.free_pages(0) == 2 and m.free_pages(1) == 4 and m.free_pages(2) == 0
    assert m.pages_needed([(a, 12, 9)]) == [3, 3, 0]
    with pytest.raises(OutOfPages) as err:
        m.reserve([(a, 12, 9)])
    assert err.value.group == "full"
    m.close(a)
    m.assert_clean()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders(seed):
    rs = np.random.RandomState(seed)
    window = [None, 5, None, 9, None, 3][seed]
    m = manager(pages=12, page_size=4, max_requests=4, max_len=40, window=window)
    live, done, next_id = {}, 0, 0
    for _ in range(400):
        action = rs.randint(0, 10)
        if action < 2 and len(live) < 4:
            live[m.open(f"r{next_id}")] = 0
            next_id += 1
        elif action < 8 and live:
            chosen = [s for s in live if rs.rand() < 0.6 and live[s] < 40] or []
            entries = [(s, live[s], int(rs.randint(1, min(9, 40 - live[s]) + 1))) for s in chosen]
            if entries:
                try:
                    res = m.reserve(entries)
                except OutOfPages:
                    m.check_invariants()
                    victim = max(live, key=lambda s: live[s])
                    if rs.rand() < 0.5:
                        m.preempt(victim)
                        live[victim] = 0
                    else:
                        m.close(victim)
                        del live[victim]
                        done += 1
                    continue
                if rs.rand() < 0.15:
                    m.rollback(res)
                else:
                    m.commit(res)
                    for s, start, count in entries:
                        live[s] = start + count
        elif live:
            s = list(live)[rs.randint(len(live))]
            m.close(s)
            del live[s]
            done += 1
        m.check_invariants()
        for s, n in live.items():
            assert m.length[s] == n
    for s in list(live):
        m.close(s)
    m.assert_clean()
    assert done > 5


def test_keys_and_values_may_differ_in_heads_and_size():
    """A mixer may keep values of another head count and size than its keys: two tensors, one page table."""
    import torch
    need = KVNeed(kv_heads=2, head_dim=24, value_heads=1, value_dim=40)
    assert (need.v_heads, need.v_dim, need.elements_per_token()) == (1, 40, 2 * 24 + 40)
    assert KVNeed(3, 16).elements_per_token() == 2 * 3 * 16
    m = CacheManager([CacheGroupSpec("odd", need, 3)], kv_pages=5, page_size=4, max_requests=2, max_len=16,
                     dtype=torch.float32, device="cpu")
    keys, values = m.kv_layer(0, 2)
    assert keys.shape == (5, 4, 2, 24) and values.shape == (5, 4, 1, 40)
    assert m.bytes_per_token() == 3 * (2 * 24 + 40) * 4


def test_pages_per_group_out_of_one_byte_budget():
    import torch
    from ayaka_py_b200.cache.manager import pages_for_budget
    full = CacheGroupSpec("full", KVNeed(4, 32), 6)                    # 6 layers, every key kept
    wide = CacheGroupSpec("wide", KVNeed(8, 64), 2)                    # 2 layers, four times the bytes per token and layer
    local = CacheGroupSpec("local", KVNeed(4, 32, window=48), 6)       # a window of 48 keys
    state = CacheGroupSpec("state", StateNeed((7,)), 2)
    kw = dict(page_size=16, max_requests=4, max_len=1024, step_tokens=64, dtype=torch.bfloat16)
    cost = lambda g: g.layers * 16 * g.need.elements_per_token() * 2
    budget = 64 << 20
    pages = pages_for_budget([full, wide, local, state], budget, **kw)
    assert pages[3] == 0
    # behind a window a request never holds more than window + one step: 4 requests x (ceil(112 / 16) + 1) pages + padding
    assert pages[2] == 4 * 8 + 1
    # the groups that keep every key hold the same number of tokens, and the budget is used but not passed
    assert pages[0] == pages[1]
    spent = sum(p * cost(g) for p, g in zip(pages[:3], (full, wide, local)))
    assert budget - (cost(full) + cost(wide)) < spent <= budget
    m = CacheManager([full, wide, local, state], kv_pages=pages, page_size=16, max_requests=4, max_len=1024, device=None)
    assert m.pages_of == pages and m.free_pages(0) == pages[0] - 1 and m.free_pages(2) == 32
    a = m.open("a")
    m.commit(m.reserve([(a, 0, 300)]))
    assert m.free_pages(0) == pages[0] - 1 - 19 and m.free_pages(1) == pages[1] - 1 - 19
    assert m.free_pages(2) == 32 - 4                                    # 300 tokens, window 48: pages 15..18 stay
    m.close(a)
    m.assert_clean()
    with pytest.raises(ValueError):
        pages_for_budget([full, wide], 1000, **kw)                      # not even one page each
    with pytest.raises(ValueError):
        CacheManager([full, wide], kv_pages=[9], page_size=16, max_requests=1, max_len=64, device=None)
