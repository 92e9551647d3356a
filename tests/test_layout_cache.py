"""The cache of captured step layouts (no GPU): capture at the second sighting, least recently
used out first, and a serving run with more layouts than room still ends up replayed."""

import random

from somi_inference_b200.engine.engine import LayoutCache


def run_layout(cache: LayoutCache, key) -> str:
    """What `Engine._run` does with a layout: replay, or run eagerly and perhaps capture."""
    if cache.get(key) is not None:
        return "replayed"
    if cache.sighted(key):
        cache.put(key, ("graph", key))
        return "captured"
    return "eager"


def test_capture_at_the_second_sighting_then_replay():
    c = LayoutCache(capacity=4)
    assert [run_layout(c, "a") for _ in range(4)] == ["eager", "captured", "replayed", "replayed"]
    assert len(c) == 1 and c.hits == 2 and c.captures == 1


def test_least_recently_used_layout_makes_room():
    c = LayoutCache(capacity=2)
    for k in ("a", "a", "b", "b"):
        run_layout(c, k)
    assert "a" in c and "b" in c
    run_layout(c, "a")                       # a is now the more recent of the two
    run_layout(c, "c")
    assert run_layout(c, "c") == "captured"  # b, used longest ago, goes
    assert "a" in c and "c" in c and "b" not in c and c.evictions == 1
    # an evicted layout starts over: eager, then captured again
    assert [run_layout(c, "b") for _ in range(3)] == ["eager", "captured", "replayed"]


def test_more_layouts_than_room_still_end_up_replayed():
    """Decode steps of a serving run: the layout is (requests, table width); requests come and
    go and contexts grow, so the run passes through several times more layouts than the cache
    holds.  Each layout lasts for many steps, so nearly every step must be a replay."""
    rng = random.Random(0)
    c = LayoutCache(capacity=8)
    outcomes = {"eager": 0, "captured": 0, "replayed": 0}
    layouts = set()
    requests, width = 4, 1
    for step in range(6000):
        if step % 40 == 39:                  # a request ends or arrives
            requests = max(1, min(16, requests + rng.choice((-1, 1))))
        if step % 150 == 149:                # the longest context crosses a width boundary
            width += 1
        key = (requests, width)
        layouts.add(key)
        outcomes[run_layout(c, key)] += 1
    assert len(layouts) > 5 * c.capacity
    assert len(c) <= c.capacity and c.evictions > 0
    assert outcomes["replayed"] > 0.9 * 6000, outcomes


def test_layouts_seen_once_do_not_pile_up():
    c = LayoutCache(capacity=2, max_sightings=10)
    for k in range(100):
        assert run_layout(c, k) == "eager"
    assert len(c._seen) <= 11 and len(c) == 0
