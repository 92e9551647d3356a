"""Scheduler decisions with a real cache manager on the CPU and no model (no GPU)."""

import pytest
import torch

from somi_inference_b200.cache import CacheManager
from somi_inference_b200.engine.scheduler import Request, RequestStatus, Scheduler
from somi_inference_b200.parts.base import CacheNeeds, PagedKVNeeds
from somi_inference_b200.sampling import SamplingParams


def make(num_pages=8, page_size=4, max_concurrent=4, budget=16, chunk=8, policy="preempt", eos=None):
    cache = CacheManager([CacheNeeds(paged=PagedKVNeeds(1, 8, None))], [None], num_pages=num_pages,
                         page_size=page_size, max_requests=max_concurrent, max_positions=64,
                         dtype=torch.float32, device="cpu")
    return cache, Scheduler(cache, max_concurrent=max_concurrent, max_num_batched_tokens=budget,
                            chunk_size=chunk, max_positions=64, eos_token_id=eos, policy=policy)


def req(i, n_prompt, max_new=4):
    return Request(i, list(range(1, n_prompt + 1)), max_new, SamplingParams(temperature=0.0))


def run_step(s, token=9):
    b = s.schedule()
    done = s.update(b, {i.request.request_id: token for i in b.items if i.samples})
    return b, done


def test_prompt_is_cut_into_portions_under_the_budget():
    cache, s = make(budget=10, chunk=6)
    s.add_request(req(0, 15))
    b, _ = run_step(s)
    assert [(i.start, i.num_tokens, i.samples) for i in b.items] == [(0, 6, False)]
    b, _ = run_step(s)
    assert [(i.start, i.num_tokens, i.samples) for i in b.items] == [(6, 6, False)]
    b, _ = run_step(s)
    assert [(i.start, i.num_tokens, i.samples) for i in b.items] == [(12, 3, True)]
    b, _ = run_step(s)                                   # now decoding
    assert [(i.start, i.num_tokens, i.samples) for i in b.items] == [(15, 1, True)]


def test_decode_tokens_come_first_and_share_the_budget():
    cache, s = make(budget=8, chunk=8, num_pages=16)
    s.add_request(req(0, 3))
    run_step(s)
    s.add_request(req(1, 20))
    b, _ = run_step(s)
    assert [(i.request.request_id, i.num_tokens) for i in b.items] == [(0, 1), (1, 7)]
    assert b.admitted and b.admitted[0].request_id == 1
    b, _ = run_step(s)
    assert [(i.request.request_id, i.num_tokens) for i in b.items] == [(0, 1), (1, 7)]


def test_finish_by_length_and_eos_frees_pages():
    cache, s = make(eos=7)
    s.add_request(req(0, 5, max_new=3))
    s.add_request(req(1, 5, max_new=3))
    run_step(s, token=9)
    assert cache.free_pages() == [4]
    b = s.schedule()
    done = s.update(b, {0: 7, 1: 9})                     # request 0 meets EOS
    assert [r.request_id for r in done] == [0] and done[0].finish_reason == "eos"
    assert done[0].output_tokens == [9, 7]               # EOS is kept
    assert cache.free_pages() == [6]
    _, done = run_step(s, token=9)
    assert [r.request_id for r in done] == [1] and done[0].finish_reason == "length"
    assert cache.free_pages() == [8] and not s.has_unfinished()
    assert [r.request_id for r in s.drain_finished()] == [0, 1] and s.drain_finished() == []


def test_ignore_eos():
    cache, s = make(eos=7)
    r = req(0, 2, max_new=3)
    r.ignore_eos = True
    s.add_request(r)
    for _ in range(3):
        run_step(s, token=7)
    assert r.status is RequestStatus.FINISHED and r.output_tokens == [7, 7, 7]


def test_max_concurrent_and_fcfs():
    cache, s = make(max_concurrent=2, num_pages=16)
    for i in range(3):
        s.add_request(req(i, 2, max_new=2))
    b, _ = run_step(s)
    assert [r.request_id for r in b.admitted] == [0, 1] and len(s.waiting) == 1
    b, done = run_step(s)
    assert len(done) == 2 and not b.admitted
    b, _ = run_step(s)
    assert [r.request_id for r in b.admitted] == [2]


def test_impossible_request_is_refused():
    cache, s = make(num_pages=4, page_size=4)
    with pytest.raises(ValueError, match="pages"):
        s.add_request(req(0, 16, max_new=2))             # 17 tokens at its longest > 16
    with pytest.raises(ValueError, match="positions"):
        s.add_request(req(1, 60, max_new=10))
    s.add_request(req(2, 13, max_new=4))                 # exactly 16 tokens: fits


def test_head_of_line_blocks_when_pages_are_short():
    cache, s = make(num_pages=4, page_size=4, budget=32, chunk=32)
    s.add_request(req(0, 10, max_new=2))
    s.add_request(req(1, 8, max_new=2))
    s.add_request(req(2, 2, max_new=2))
    b, _ = run_step(s)
    assert [r.request_id for r in b.admitted] == [0]     # 1 needs 2 pages, 1 is free; 2 waits behind it
    assert [r.request_id for r in s.waiting] == [1, 2]


def test_preemption_by_recompute_when_pages_run_out():
    cache, s = make(num_pages=4, page_size=4, budget=32, chunk=32)
    a, b_ = req(0, 7, max_new=8), req(1, 7, max_new=8)
    s.add_request(a)
    s.add_request(b_)
    run_step(s)                                          # both prefilled: 2 pages each, pool empty
    assert cache.free_pages() == [0]
    batch, _ = run_step(s)                               # both decode into their 8th slot
    assert not batch.preempted
    batch = s.schedule()                                 # position 8 needs a third page each
    assert [r.request_id for r in batch.preempted] == [1]   # the most recently admitted goes
    assert [i.request.request_id for i in batch.items] == [0]
    assert b_.status is RequestStatus.WAITING and b_.num_computed == 0 and b_.num_preemptions == 1
    assert s.waiting[0] is b_ and len(b_.output_tokens) == 2
    assert not cache.is_registered(1)
    s.update(batch, {0: 9})
    cache.check_consistency()
    # request 0 runs to its end; then request 1 is readmitted and recomputes prompt + 2 outputs
    while a.status is not RequestStatus.FINISHED:
        run_step(s)
    batch, _ = run_step(s)
    assert [r.request_id for r in batch.admitted] == [1]
    assert [(i.start, i.num_tokens, i.samples) for i in batch.items] == [(0, 9, True)]
    while s.has_unfinished():
        run_step(s)
    assert len(b_.output_tokens) == 8 and cache.free_pages() == [4]


def test_reserve_policy_never_preempts():
    cache, s = make(num_pages=4, page_size=4, budget=32, chunk=32, policy="reserve")
    a, b_ = req(0, 7, max_new=8), req(1, 7, max_new=8)      # 14 tokens at most: 4 pages each
    s.add_request(a)
    s.add_request(b_)
    batch, _ = run_step(s)
    assert [r.request_id for r in batch.admitted] == [0]    # the worst case of both does not fit
    preempted = 0
    while s.has_unfinished():
        batch, _ = run_step(s)
        preempted += len(batch.preempted)
    assert preempted == 0 and len(a.output_tokens) == 8 and len(b_.output_tokens) == 8


def test_request_validation():
    with pytest.raises(ValueError):
        Request(0, [1], 0)
    with pytest.raises(ValueError):
        Request(0, [], 3)
    for bad in (dict(temperature=-1.0), dict(top_k=0), dict(top_p=0.0), dict(top_p=1.5),
                dict(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_the_next_decode_step_decided_early_is_what_schedule_would_decide():
    """`continue_decoding` after `advance`: the same items and the same pages as `schedule()`
    gives after `update`, in two schedulers fed the same way."""
    outs = []
    for early in (False, True):
        cache, s = make(num_pages=12, eos=7)
        for i, n in enumerate([5, 3, 6]):
            s.add_request(req(i, n, max_new=6))
        log = []
        b = s.schedule()
        nxt = None
        for step in range(8):
            toks = {i.request.request_id: 9 for i in b.items if i.samples}
            if early:
                s.advance(b)
                nxt = s.continue_decoding() if all(i.samples for i in b.items) else None
                s.update(b, toks, advanced=True)
            else:
                s.update(b, toks)
            if not s.has_unfinished():
                break
            if nxt is not None and s.still_valid(nxt):
                b = nxt
            else:
                if nxt is not None:
                    s.abandon(nxt)
                b = s.schedule()
            nxt = None
            log.append(([(i.request.request_id, i.start, i.num_tokens, i.samples) for i in b.items],
                        cache.free_pages()))
            cache.check_consistency()
        outs.append(log)
    assert outs[0] == outs[1] and len(outs[0]) >= 4


def test_early_decision_is_given_back_when_a_request_ends_or_arrives():
    cache, s = make(num_pages=12, eos=7)
    s.add_request(req(0, 4, max_new=8))
    s.add_request(req(1, 4, max_new=8))
    b = s.schedule()
    s.advance(b)
    nxt = s.continue_decoding()
    assert nxt is not None and [i.request.request_id for i in nxt.items] == [0, 1]
    assert all(i.num_tokens == 1 and i.samples and i.start == 4 for i in nxt.items)
    free_with_reservation = cache.free_pages()
    # request 0 meets the end-of-sequence token on the token that arrives now
    done = s.update(b, {0: 7, 1: 9}, advanced=True)
    assert [r.request_id for r in done] == [0] and not s.still_valid(nxt)
    s.abandon(nxt)
    cache.check_consistency()
    b2 = s.schedule()
    assert [(i.request.request_id, i.start, i.num_tokens) for i in b2.items] == [(1, 4, 1)]
    s.update(b2, {1: 9})
    # a request that arrives makes the early decision void as well
    b3 = s.schedule()
    s.advance(b3)
    nxt = s.continue_decoding()
    assert nxt is not None
    s.update(b3, {1: 9}, advanced=True)
    s.add_request(req(2, 3))
    assert not s.still_valid(nxt)
    s.abandon(nxt)
    cache.check_consistency()
    assert free_with_reservation is not None


def test_no_early_decision_when_it_would_depend_on_the_token():
    cache, s = make(num_pages=12)
    s.add_request(req(0, 4, max_new=2))
    s.add_request(req(1, 12, max_new=4))
    b = s.schedule()                       # request 1 has a portion of its prompt left
    s.advance(b)
    assert s.continue_decoding() is None   # not every running request is about to decode
    s.update(b, {0: 9}, advanced=True)
    b = s.schedule()
    s.advance(b)
    assert s.continue_decoding() is None   # request 0 ends by length on the token that arrives
    s.update(b, {0: 9, 1: 9}, advanced=True)
    # no page left for another token: left to schedule(), which may preempt
    cache2, s2 = make(num_pages=2, page_size=4)
    s2.add_request(req(0, 4, max_new=4))
    s2.add_request(req(1, 4, max_new=4))
    b = s2.schedule()
    s2.advance(b)
    assert s2.continue_decoding() is None and cache2.free_pages() == [0]
    cache2.check_consistency()


def test_abort_gives_everything_back_whatever_the_state():
    cache, s = make(num_pages=8, page_size=4, max_concurrent=2)
    a, b, c = req(0, 6, max_new=8), req(1, 5, max_new=8), req(2, 3, max_new=8)
    for r in (a, b, c):
        s.add_request(r)
    run_step(s)                                          # a and b run, c waits
    assert [r.request_id for r in s.running] == [0, 1] and list(s.waiting) == [c]
    assert s.abort(c) and c.status is RequestStatus.FINISHED and c.finish_reason == "aborted"
    assert not s.waiting
    # b is aborted while the next decode step is decided and its page reserved
    run_step(s)
    nxt = s.schedule()
    s.advance(nxt)
    early = s.continue_decoding()
    assert early is not None and len(early.items) == 2
    s.update(nxt, {0: 9, 1: 9}, advanced=True)
    assert s.abort(b)
    assert not s.still_valid(early)
    s.abandon(early)
    cache.check_consistency()
    assert [r.request_id for r in s.running] == [0]
    assert not s.abort(b)                                 # already out
    assert not s.abort(req(7, 3))                         # never added
    while s.has_unfinished():
        run_step(s)
    assert cache.free_pages() == [8]
    assert {r.request_id for r in s.drain_finished()} == {0, 1, 2}


def test_no_decoder_waits_for_another_requests_prompt():
    """A long prompt admitted before three decoding requests must not take their tokens: with a
    budget of 10 and portions of 8, each decoder gets its token in every step and the prompt
    takes what is left (continuous_batching.py:91 decodes every running sequence every step)."""
    cache, s = make(num_pages=64, budget=10, chunk=8, max_concurrent=8)
    long = req(0, 40, max_new=2)
    s.add_request(long)
    run_step(s)                                          # first portion of the long prompt
    for i in (1, 2, 3):
        s.add_request(req(i, 2, max_new=12))
    s.max_num_batched_tokens = 32
    run_step(s)                                          # admitted, their prompts computed
    s.max_num_batched_tokens = 10
    assert [r.request_id for r in s.running] == [0, 1, 2, 3]
    while long.num_computed < len(long.prompt_tokens):
        left = len(long.prompt_tokens) - long.num_computed
        b, _ = run_step(s)
        got = {i.request.request_id: i.num_tokens for i in b.items}
        assert got[1] == got[2] == got[3] == 1, got       # nobody skips a step
        assert got[0] == min(7, left), got                # the prompt takes the rest of the budget
        assert [i.request.request_id for i in b.items][:3] == [1, 2, 3]


def test_budget_of_a_preempted_request_goes_back():
    """The victim of a preemption may already have its token in the step (decoders are served
    before portions): its item is dropped and its token is not charged to the budget."""
    cache, s = make(num_pages=6, page_size=4, budget=6, chunk=4, max_concurrent=4)
    a, b_ = req(0, 20, max_new=2), req(1, 2, max_new=8)
    s.add_request(a)
    s.add_request(b_)
    for _ in range(4):
        batch, _ = run_step(s)
        assert not batch.preempted
    assert cache.free_pages() == [0] and a.num_computed == 16 and b_.num_tokens == 6
    batch = s.schedule()          # b's token first, then a's last portion needs a page: b goes
    assert [r.request_id for r in batch.preempted] == [1]
    assert [(i.request.request_id, i.num_tokens) for i in batch.items] == [(0, 4)]
    assert b_.num_computed == 0 and s.waiting[0] is b_
    s.update(batch, {0: 9})
    cache.check_consistency()
    while s.has_unfinished():
        run_step(s)
    assert len(a.output_tokens) == 2 and len(b_.output_tokens) == 8
    assert cache.free_pages() == [6]


def make_windowed(window, num_pages, page_size=4, chunk=4, policy="preempt", positions=256):
    cache = CacheManager([CacheNeeds(paged=PagedKVNeeds(1, 8, window))], [None],
                         num_pages=num_pages, page_size=page_size, max_requests=4,
                         max_positions=positions, dtype=torch.float32, device="cpu")
    return cache, Scheduler(cache, max_concurrent=4, max_num_batched_tokens=16, chunk_size=chunk,
                            max_positions=positions, policy=policy)


@pytest.mark.parametrize("policy", ["preempt", "reserve"])
def test_windowed_model_is_admitted_where_the_window_fits(policy):
    """A request far longer than the pool is admitted when every layer reads a window only: it
    never holds more than ceil((window + portion) / page) + 1 pages."""
    cache, s = make_windowed(window=8, num_pages=5, policy=policy)
    r = req(0, 60, max_new=30)                            # 89 positions = 23 pages if all were kept
    s.add_request(r)
    most = 0
    while s.has_unfinished():
        b, _ = run_step(s)
        assert not b.preempted
        most = max(most, 5 - cache.free_pages()[0])
        cache.check_consistency()
    assert r.status is RequestStatus.FINISHED and len(r.output_tokens) == 30
    assert most <= 4
    # without a window the same request is refused
    _, s2 = make(num_pages=5, page_size=4)
    s2.max_positions = 256
    with pytest.raises(ValueError):
        s2.add_request(req(0, 60, max_new=30))


def test_reserve_policy_counts_windowed_requests_by_their_window():
    cache, s = make_windowed(window=8, num_pages=8, policy="reserve")
    for i in range(3):
        s.add_request(req(i, 30, max_new=10))
    b, _ = run_step(s)
    # each request reserves ceil((8 + 4) / 4) + 1 = 4 pages: two fit into 8 pages, the third waits
    assert [r.request_id for r in b.admitted] == [0, 1] and len(s.waiting) == 1


@pytest.mark.parametrize("policy", ["preempt", "reserve"])
def test_model_with_fixed_state_only(policy):
    """A model whose mixers keep only fixed-size state has no page group: admission is bounded by
    the slots alone, under both policies."""
    from somi_inference_b200.parts.base import StateNeeds
    cache = CacheManager([CacheNeeds(state=StateNeeds({"s": ((4,), torch.float32)}))], [None],
                         num_pages=1, page_size=4, max_requests=2, max_positions=64,
                         dtype=torch.float32, device="cpu")
    s = Scheduler(cache, max_concurrent=4, max_num_batched_tokens=16, chunk_size=8,
                  max_positions=64, policy=policy)
    assert cache.groups == []
    for i in range(3):
        s.add_request(req(i, 5, max_new=3))
    done = []
    for _ in range(20):
        if not s.has_unfinished():
            break
        _, d = run_step(s)
        done += d
    assert sorted(r.request_id for r in done) == [0, 1, 2]
