"""Continuous-batching scheduler: admission, prompt portions under a token budget, decode,
finish, and what happens when pages run out.

The reference's scheduler (somi_inference/core/continuous_batching.py:46-120) is
first-come-first-served over three queues, admits a sequence only if its
worst-case block count ceil((prompt + max_new - 1) / block_size) fits beside the
reservations of everything running (:64-67, :92-104), runs whole prompts, and so
never runs out of blocks; a request larger than the pool blocks the queue for
ever (:97-98).  This scheduler keeps the three queues, the FCFS order with
head-of-line blocking, the finish rule (EOS or max_new_tokens, EOS kept in the
output: :150-158) and `max_concurrent`, and adds:

* a token budget per step and prompt portions of at most `chunk_size` tokens,
  scheduled beside the single decode tokens of running requests; the decode tokens are
  served first (no running request that decodes waits for another one's prompt), portions
  share what is left of the budget;
* pages are taken per step for exactly the scheduled tokens.  Policy "preempt"
  (default): when a running request cannot get a page, the most recently
  admitted running request is preempted by recompute: its pages go back, it
  returns to the front of the waiting queue, and its prompt plus the tokens it
  has generated are computed again when it is readmitted.  Policy "reserve":
  the reference's worst-case reservation at admission, under which pages cannot
  run out;
* a request that could never fit (pool or position limit) is refused by
  `add_request` with a ValueError instead of blocking the queue.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from enum import Enum

from ..cache import OutOfPages
from ..sampling import SamplingParams


class RequestStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class Request:
    request_id: int
    prompt_tokens: list[int]
    max_new_tokens: int
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    ignore_eos: bool = False
    seed: int = 0
    status: RequestStatus = RequestStatus.WAITING
    output_tokens: list[int] = field(default_factory=list)
    num_computed: int = 0          # tokens whose keys/values are in the cache
    num_preemptions: int = 0
    finish_reason: str | None = None

    def __post_init__(self) -> None:
        if self.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be > 0")
        if not self.prompt_tokens:
            raise ValueError("a request needs at least one prompt token")

    @property
    def all_tokens(self) -> list[int]:
        return self.prompt_tokens + self.output_tokens

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_tokens) + len(self.output_tokens)

    def tokens(self, start: int, n: int) -> list[int]:
        """Tokens [start, start + n) of prompt + output, without joining the two lists."""
        p = len(self.prompt_tokens)
        if start >= p:
            return self.output_tokens[start - p:start - p + n]
        if start + n <= p:
            return self.prompt_tokens[start:start + n]
        return self.prompt_tokens[start:] + self.output_tokens[:start + n - p]


@dataclass
class ScheduledItem:
    request: Request
    start: int            # index of the first token of the portion in request.all_tokens
    num_tokens: int
    samples: bool         # the portion reaches the request's last known token


@dataclass
class ScheduledBatch:
    items: list[ScheduledItem]
    preempted: list[Request]
    admitted: list[Request]

    @property
    def num_tokens(self) -> int:
        return sum(i.num_tokens for i in self.items)


class Scheduler:
    def __init__(self, cache, *, max_concurrent: int, max_num_batched_tokens: int,
                 chunk_size: int, max_positions: int, eos_token_id: int | None = None,
                 policy: str = "preempt") -> None:
        if policy not in ("preempt", "reserve"):
            raise ValueError("policy must be 'preempt' or 'reserve'")
        if max_num_batched_tokens < 1 or chunk_size < 1 or max_concurrent < 1:
            raise ValueError("max_concurrent, max_num_batched_tokens and chunk_size must be >= 1")
        self.cache = cache
        self.max_concurrent = max_concurrent
        self.max_num_batched_tokens = max_num_batched_tokens
        self.chunk_size = chunk_size
        self.max_positions = max_positions
        self.eos_token_id = eos_token_id
        self.policy = policy
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []

    # --------------------------------------------------------------- requests
    def _pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.cache.page_size)

    def _worst_case_pages(self, req: Request) -> list[int]:
        """For every group of the cache, the most pages the request can hold at a time.  A group
        that keeps all keys: ceil((prompt + max_new - 1) / page_size), as
        continuous_batching.py:64-67.  A group with a window of w keeps the pages between the
        oldest key a query still reads and the end of the portion being written: at most
        ceil((w + portion) / page_size) + 1, whatever the length."""
        full = self._pages_for(len(req.prompt_tokens) + req.max_new_tokens - 1)
        out = []
        for g in self.cache.groups:
            w = g.needs.window
            if w is None:
                out.append(full)
            else:
                out.append(min(full, self._pages_for(w + self.chunk_size) + 1))
        return out

    def add_request(self, req: Request) -> None:
        most = len(req.prompt_tokens) + req.max_new_tokens - 1
        if most > self.max_positions:
            raise ValueError(f"request {req.request_id}: prompt + max_new_tokens - 1 = {most} "
                             f"exceeds the model's {self.max_positions} positions")
        for g, need in zip(self.cache.groups, self._worst_case_pages(req)):
            if need > g.pool.num_pages:
                raise ValueError(f"request {req.request_id} needs {need} pages at its longest; "
                                 f"the cache has {g.pool.num_pages}"
                                 + (f" (window {g.needs.window})" if g.needs.window else ""))
        req.status = RequestStatus.WAITING
        self.waiting.append(req)

    def abort(self, req: Request) -> bool:
        """Take a request out, whatever its state: what it holds in the cache (reserved pages of a
        step that is prepared or on its way included) goes back at once.  Returns whether it was
        still unfinished.  (The reference has no such call; a caller that stops reading a stream
        needs it.)"""
        if req.status is RequestStatus.FINISHED:
            return False
        if req in self.running:
            self.running.remove(req)
        else:
            try:
                self.waiting.remove(req)
            except ValueError:
                return False                      # never added
        if self.cache.is_registered(req.request_id):
            self.cache.release(req.request_id)
        req.status = RequestStatus.FINISHED
        req.finish_reason = "aborted"
        self.finished.append(req)
        return True

    def has_unfinished(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def drain_finished(self) -> list[Request]:
        done, self.finished = self.finished, []
        return done

    # --------------------------------------------------------------- schedule
    def _preempt(self, victim: Request, items: list[ScheduledItem],
                 preempted: list[Request]) -> int:
        """Take `victim` out by recompute; returns the tokens of the step that it gives back."""
        self.cache.release(victim.request_id)
        self.running.remove(victim)
        given_back = sum(i.num_tokens for i in items if i.request is victim)
        items[:] = [i for i in items if i.request is not victim]
        victim.status = RequestStatus.WAITING
        victim.num_computed = 0
        victim.num_preemptions += 1
        self.waiting.appendleft(victim)
        preempted.append(victim)
        return given_back

    def schedule(self) -> ScheduledBatch:
        budget = self.max_num_batched_tokens
        items: list[ScheduledItem] = []
        preempted: list[Request] = []
        admitted: list[Request] = []

        def serve(req: Request, n: int) -> int:
            """Reserve `n` tokens for a running request, preempting from the back of the line
            while pages are missing; returns the change of the budget."""
            back = 0
            while True:
                try:
                    self.cache.reserve(req.request_id, n)
                    break
                except OutOfPages:
                    victim = self.running[-1]
                    back += self._preempt(victim, items, preempted)
                    if victim is req:
                        return back
            items.append(ScheduledItem(req, req.num_computed, n, req.num_computed + n == req.num_tokens))
            return back - n

        # 1. every running request that decodes gets its one token first, in admission order
        #    (continuous_batching.py:91 decodes every running sequence in every step) ...
        for req in list(self.running):
            if budget <= 0:
                break
            if req in self.running and req.num_tokens - req.num_computed == 1:
                budget += serve(req, 1)
        # ... then the requests that are still in their prompt (or recomputing after a
        # preemption) share what is left, in portions
        for req in list(self.running):
            if budget <= 0:
                break
            left = req.num_tokens - req.num_computed
            if req in self.running and left > 1 and not any(i.request is req for i in items):
                budget += serve(req, min(left, self.chunk_size, budget))

        # 2. admission, first come first served, head of the line blocks
        reserved_worst = [0] * len(self.cache.groups)
        if self.policy == "reserve":
            for r in self.running:
                reserved_worst = [a + b for a, b in zip(reserved_worst, self._worst_case_pages(r))]
        while (self.waiting and len(self.running) < self.max_concurrent and budget > 0
               and not preempted):
            req = self.waiting[0]
            n = min(req.num_tokens - req.num_computed, self.chunk_size, budget)
            if self.policy == "reserve":
                worst = self._worst_case_pages(req)
                if any(a + b > g.pool.num_pages
                       for a, b, g in zip(reserved_worst, worst, self.cache.groups)):
                    break
                reserved_worst = [a + b for a, b in zip(reserved_worst, worst)]
            try:
                self.cache.register(req.request_id)
            except OutOfPages:                 # every state slot of the cache is taken
                break
            try:
                self.cache.reserve(req.request_id, n)
            except OutOfPages:
                self.cache.release(req.request_id)
                break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            admitted.append(req)
            items.append(ScheduledItem(req, req.num_computed, n, req.num_computed + n == req.num_tokens))
            budget -= n
        return ScheduledBatch(items, preempted, admitted)

    # ------------------------------------------------- the next step, early
    def advance(self, batch: ScheduledBatch) -> None:
        """The part of `update` that needs no sampled token: the step's tokens are in the cache."""
        for item in batch.items:
            self.cache.commit(item.request.request_id)
            item.request.num_computed += item.num_tokens

    def continue_decoding(self) -> ScheduledBatch | None:
        """The next step's schedule, decided while the tokens of this step are still being
        sampled, for the one state in which it does not depend on them: nobody waits, and every
        running request has just had its last known token computed and cannot finish by length
        on the token that is about to arrive.  `schedule()` would then give every running request
        one decode token, in order, and nothing else; that is what is reserved and returned here.
        None where the state is another one, or where a page is missing (then `schedule()`
        decides, with preemption if it must).  Call after `advance`; if a request finishes on
        the arriving token after all (end of sequence), `abandon` the batch.
        """
        if self.waiting or not self.running or len(self.running) > self.max_num_batched_tokens:
            return None
        for req in self.running:
            if req.num_computed != req.num_tokens or len(req.output_tokens) + 1 >= req.max_new_tokens:
                return None
        reserved: list[Request] = []
        try:
            for req in self.running:
                self.cache.reserve(req.request_id, 1)
                reserved.append(req)
        except OutOfPages:
            for req in reserved:
                self.cache.cancel(req.request_id)
            return None
        # the token itself sits at index num_computed once it has arrived
        return ScheduledBatch([ScheduledItem(r, r.num_computed, 1, True) for r in self.running], [], [])

    def still_valid(self, batch: ScheduledBatch) -> bool:
        """Whether a batch from `continue_decoding` is what `schedule()` would decide now."""
        return (not self.waiting and len(batch.items) == len(self.running)
                and all(i.request is r for i, r in zip(batch.items, self.running)))

    def abandon(self, batch: ScheduledBatch) -> None:
        """Give back what `continue_decoding` reserved (requests that ended meanwhile have
        given everything back already)."""
        for item in batch.items:
            if self.cache.is_registered(item.request.request_id):
                self.cache.cancel(item.request.request_id)

    # ----------------------------------------------------------------- update
    def update(self, batch: ScheduledBatch, sampled: dict[int, int],
               advanced: bool = False) -> list[Request]:
        """After the step: advance (unless `advance` was called already), append sampled
        tokens, finish and free.

        `sampled` maps request_id to the token sampled for every item with
        `samples`.  Returns the requests that finished in this step.
        """
        done: list[Request] = []
        if not advanced:
            self.advance(batch)
        for item in batch.items:
            req = item.request
            if not item.samples:
                continue
            token = int(sampled[req.request_id])
            req.output_tokens.append(token)
            hit_eos = (not req.ignore_eos and self.eos_token_id is not None
                       and token == self.eos_token_id)
            if hit_eos or len(req.output_tokens) >= req.max_new_tokens:
                req.status = RequestStatus.FINISHED
                req.finish_reason = "eos" if hit_eos else "length"
                self.cache.release(req.request_id)
                self.running.remove(req)
                self.finished.append(req)
                done.append(req)
        return done
