"""Cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; state slots; all-or-nothing reservation (no GPU)."""

import random

import pytest
import torch

from somi_inference_b200.cache import FREED, CacheManager, OutOfPages, PagePool
from somi_inference_b200.parts.base import CacheNeeds, PagedKVNeeds, StateNeeds


def manager(num_pages=10, page_size=4, windows=(None,), max_requests=5, state=False, runs=2):
    needs = []
    for w in windows:
        for _ in range(runs):
            needs.append(CacheNeeds(paged=PagedKVNeeds(2, 8, w),
                                    state=StateNeeds({"h": ((3,), torch.float32)}) if state else None))
    return CacheManager(needs, [None] * len(needs), num_pages=num_pages, page_size=page_size,
                        max_requests=max_requests, max_positions=200, dtype=torch.float32,
                        device="cpu")


def test_pool_refuses_misuse():
    p = PagePool(3)
    a = p.take(2)
    assert a == [0, 1] and p.num_free == 1
    with pytest.raises(OutOfPages):
        p.take(2)
    assert p.num_free == 1                      # nothing was taken by the failed call
    p.give_back([a[0]])
    with pytest.raises(RuntimeError, match="not held"):
        p.give_back([a[0]])                     # freed twice
    with pytest.raises(ValueError):
        p.give_back([7])
    assert p.take(1) == [a[0]]                  # last given back is handed out first


def test_groups_by_needs():
    m = manager(windows=(None, 6, None))
    assert len(m.groups) == 2                   # two full-attention specs share one group
    assert [len(g.runs) for g in m.groups] == [4, 2]
    assert m.groups[0].storage.shape == (4, 2, 10, 2, 4, 8)
    assert m.view(0).paged.group == 0 and m.view(2).paged.group == 1 and m.view(4).paged.group == 0
    assert m.view(0).paged.keys.data_ptr() != m.view(1).paged.keys.data_ptr()


def test_reserve_commit_release():
    m = manager()
    m.register("a")
    with pytest.raises(ValueError):
        m.register("a")
    m.reserve("a", 5)
    assert m.free_pages() == [8]
    with pytest.raises(RuntimeError, match="uncommitted"):
        m.reserve("a", 1)
    m.commit("a")
    assert m.length("a") == 5
    m.reserve("a", 3)                           # positions 5..7 fit in the second page
    assert m.free_pages() == [8]
    m.commit("a")
    m.reserve("a", 1)
    assert m.free_pages() == [7]
    m.cancel("a")
    assert m.free_pages() == [8] and m.length("a") == 8
    m.check_consistency()
    m.release("a")
    assert m.free_pages() == [10]
    with pytest.raises(KeyError):
        m.release("a")


def test_all_or_nothing_across_groups():
    m = manager(num_pages=4, windows=(None, 4))
    m.register("a")
    m.reserve("a", 12)                          # 3 pages in each group
    m.commit("a")                               # the window group keeps only what it still reads
    assert m.free_pages()[0] == 1 and m.free_pages()[1] >= 2
    m.register("b")
    before = m.free_pages()
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)                       # full group has 1 page, needs 2
    assert m.free_pages() == before             # the window group took nothing either
    m.check_consistency()


def test_window_gives_pages_back_and_marks_table():
    m = manager(num_pages=6, page_size=4, windows=(5,), runs=1)
    m.register("a")
    held_max = 0
    for step in range(40):
        m.reserve("a", 1)
        m.commit("a")
        held_max = max(held_max, 6 - m.free_pages()[0])
        L = m.length("a")
        table = m.groups[0].tables[m.slot("a")]
        first_needed = max(0, L - 5 + 1) // 4
        assert (table[:first_needed] == FREED).all()
        assert (table[first_needed:-(-L // 4)] >= 0).all()
        m.check_consistency()
    assert held_max <= 3                        # a 5-token window never spans more than 3 pages
    m.release("a")
    assert m.free_pages() == [6]


def test_state_slots_are_zeroed_and_reused():
    m = manager(state=True, max_requests=2)
    s = m.register("a")
    m.view(0).state["h"][s] = 7.0
    m.register("b")
    with pytest.raises(OutOfPages, match="request slots"):
        m.register("c")
    m.release("a")
    s2 = m.register("c")
    assert s2 == s and float(m.view(0).state["h"][s2].abs().sum()) == 0.0
    assert m.view(0).state["h"].data_ptr() != m.view(1).state["h"].data_ptr()


def test_reader_runs_share_the_owners_view():
    needs = [CacheNeeds(paged=PagedKVNeeds(2, 8, None))] * 3
    m = CacheManager(needs, [None, None, 0], num_pages=4, page_size=4, max_requests=2,
                     max_positions=16, dtype=torch.float32, device="cpu")
    assert m.view(2) is m.view(0)
    assert m.groups[0].storage.shape[0] == 2    # the reader owns no storage


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = manager(num_pages=24, page_size=4, windows=(None, 9), max_requests=6)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 6:
            m.register(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.85 and live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 11])
            before = m.free_pages()
            try:
                m.reserve(r, n)
            except OutOfPages:
                assert m.free_pages() == before
                victim = max(live, key=lambda k: live[k])
                m.release(victim)
                del live[victim]
            else:
                if rng.random() < 0.1:
                    m.cancel(r)
                else:
                    m.commit(r)
                    live[r] += n
                assert m.length(r) == live[r]
        elif live:
            r = rng.choice(list(live))
            m.release(r)
            del live[r]
        m.check_consistency()
        for r, n in live.items():
            assert len(m.held_pages(r, 0)) == -(-n // 4)
    for r in list(live):
        m.release(r)
    assert m.free_pages() == [24, 24]


def test_what_a_request_would_need_and_what_it_holds():
    """The questions a scheduler may ask before it reserves: pages a request would need for more
    tokens (per group, a windowed group counting only what its window keeps), who is live, and
    how many table entries a slot uses."""
    m = manager(num_pages=12, page_size=4, windows=(None, 6))
    m.register("a")
    assert m.live_requests() == ["a"]
    assert m.pages_needed("a", 9) == [3, 3]
    m.reserve("a", 9)
    m.commit("a")
    slot = m.slot("a")
    assert m.blocks_in_use(0, slot) == 3 and m.blocks_in_use(1, slot) == 3
    # five more tokens: positions 9..13 need one more page of four (page 2 has room for 9..11)
    assert m.pages_needed("a", 5)[0] == 1
    m.reserve("a", 5)
    m.commit("a")
    # the windowed group has given back the pages that positions 14 - 6 + 1 = 9.. no longer read
    assert len(m.held_pages("a", 1)) < len(m.held_pages("a", 0)) == 4
    m.register("b")
    assert sorted(m.live_requests()) == ["a", "b"]
    m.release("a")
    assert m.live_requests() == ["b"]
    m.check_consistency()
