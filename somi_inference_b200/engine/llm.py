"""The Python entry point: `LLM(model, ...).generate(prompt, max_new_tokens=...)`.

Names and meanings of the options follow the reference's `LLM`
(somi_inference/entrypoints/llm.py:58-70,126-135): `num_blocks`, `block_size`,
`max_concurrent`, `device`, `dtype`, and for `generate`: `max_new_tokens`,
`temperature`, `top_k`, `top_p`, `repetition_penalty`.  The reference takes a
hub model name and a text prompt and returns text; here `model` is a folder
(config.json + safetensors), a prompt may be a list of token ids (returned:
list of new token ids) or, when the folder holds tokenizer files, a string
(returned: the new text only, as llm.py:164).  Its three backend selectors do
not exist: there is one implementation.  The loop below is the reference's
`ContinuousBatchingEngine.run` (somi_inference/core/continuous_batching.py:179-205)
over one mixed batch per step instead of separate prefill and decode passes.
"""

from __future__ import annotations

import os
import random
from collections import deque
from dataclasses import dataclass
from typing import Iterator, Sequence

import torch

from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .engine import Engine
from .scheduler import Request, RequestStatus, ScheduledBatch, Scheduler

DEFAULT_BLOCK_SIZE = 16        # somi_inference/entrypoints/llm.py:25
DEFAULT_MAX_CONCURRENT = 16    # somi_inference/entrypoints/llm.py:26
DEFAULT_NUM_BLOCKS = 256       # somi_inference/entrypoints/llm.py:62


class _NoEvent:
    """Stands in for a CUDA event where the engine's device has no streams."""

    def record(self) -> None:
        pass

    def synchronize(self) -> None:
        pass


@dataclass
class _Launched:
    """A step that has been launched and whose sampled ids have not been read yet."""

    batch: ScheduledBatch
    samplers: list            # the requests that sample in it, in the order of the ids
    ids: "torch.Tensor | None"         # int32 on the device, one per sampler of the launch
    host: "torch.Tensor | None"        # the pinned copy that `event` guards
    event: object
    rows: list                # for each sampler its row among the launch's ids
    whole: bool               # no request of the launch has ended since


class LLM:
    def __init__(self, model: "str | Engine", *, num_blocks: int = DEFAULT_NUM_BLOCKS,
                 block_size: int = DEFAULT_BLOCK_SIZE,
                 max_concurrent: int = DEFAULT_MAX_CONCURRENT,
                 device: torch.device | str | None = None, dtype="float32",
                 max_num_batched_tokens: int = 2048, chunk_size: int = 512,
                 policy: str = "preempt", eos_token_id: int | None = None, ops=None) -> None:
        self.device = torch.device(device) if device is not None else torch.device("cuda:0")
        if isinstance(model, Engine):         # an engine that was built elsewhere (benchmarks)
            self.engine = model
            self.device = model.device
        else:
            self.engine = Engine(model, dtype=dtype, page_size=block_size, num_pages=num_blocks,
                                 max_requests=max_concurrent, device=self.device, ops=ops)
        self.config = self.engine.config
        if eos_token_id is None:
            eos_token_id = getattr(self.config, "eos_token_id", None)
        self.eos_token_id = eos_token_id
        self.scheduler = Scheduler(self.engine.cache, max_concurrent=max_concurrent,
                                   max_num_batched_tokens=max_num_batched_tokens,
                                   chunk_size=chunk_size,
                                   max_positions=self.engine.spec.max_positions,
                                   eos_token_id=eos_token_id, policy=policy)
        self.sampler = Sampler(self.engine.ops, self.device)
        self._next_request_id = 0
        self._tokenizer = None
        self._model_dir = model
        self.steps_run = 0
        self.d2h_bytes_last = 0
        self.prepare_early = True      # prepare the next decode step while the GPU runs this one
        self._early = None             # (scheduled batch, its descriptor) prepared for the next step
        self.run_ahead = True          # launch the next decode step before the host has the ids
        self._ahead: _Launched | None = None       # the step that was launched ahead
        self.rows_dropped = 0          # rows of steps launched ahead whose request had ended
        self._ids_host = [None, None]
        self._ids_event = [None, None]
        self._ids_turn = 0

    def sampler_h2d_bytes(self) -> int:
        return self.sampler.h2d_bytes_last

    # -------------------------------------------------------------- tokenizer
    def _tok(self):
        if self._tokenizer is None:
            if not isinstance(self._model_dir, (str, os.PathLike)):
                raise ValueError("this engine was built from tensors and has no tokenizer: give "
                                 "prompts as token ids")
            if not any(os.path.isfile(os.path.join(self._model_dir, f))
                       for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
                raise ValueError("this model folder holds no tokenizer: give prompts as token ids")
            from transformers import AutoTokenizer   # tokenizer only; no model code is used
            self._tokenizer = AutoTokenizer.from_pretrained(self._model_dir, local_files_only=True)
        return self._tokenizer

    # --------------------------------------------------------------- requests
    def make_request(self, prompt_tokens: Sequence[int], *, max_new_tokens: int,
                     sampling_params: SamplingParams | None = None,
                     ignore_eos: bool = False) -> Request:
        sp = sampling_params or SamplingParams()
        seed = sp.seed if sp.seed is not None else random.getrandbits(63)
        req = Request(self._next_request_id, list(prompt_tokens), max_new_tokens, sp,
                      ignore_eos=ignore_eos, seed=int(seed))
        self._next_request_id += 1
        return req

    # ------------------------------------------------------------------- loop
    def step(self) -> list[Request]:
        """One scheduling step and one model step; returns the requests that finished in it.

        While the GPU runs a step of single decode tokens, the next step is prepared as far as
        it does not depend on the tokens being sampled: the scheduler's decision, the pages and
        the batch descriptor (`Scheduler.continue_decoding`, `Engine.prebuild`).  Where the
        sampler needs nothing else of those tokens (no repetition penalty), the next step is
        also launched, with the sampled ids copied into its descriptor on the device, before the
        host reads them: the GPU does not wait for the host between decode steps.  Such a step is
        never taken back.  If a request ends on a token that the host sees only afterwards (end
        of sequence), its row of the step that ran ahead is dropped; a request that arrived
        meanwhile is admitted one step later.  Where the next step cannot be launched, its
        preparation is kept for the next call and given back if the state has changed by then.
        """
        cur, self._ahead = self._ahead, None
        if cur is not None:
            live = [k for k, item in enumerate(cur.batch.items)
                    if item.request.status is not RequestStatus.FINISHED]
            self.rows_dropped += len(cur.batch.items) - len(live)
            if not live:
                cur = None                   # every request of the step that ran ahead has ended
            elif len(live) < len(cur.batch.items):
                cur = _Launched(ScheduledBatch([cur.batch.items[k] for k in live], [], []),
                                [cur.samplers[k] for k in live], cur.ids, cur.host, cur.event,
                                live, False)
        if cur is None:
            cur = self._launch_next()
            if cur is None:
                return []
        batch, samplers = cur.batch, cur.samplers
        # the GPU is busy with the step: the host's part of the next one
        self.scheduler.advance(batch)
        failed_ahead: Exception | None = None
        if self.prepare_early and cur.whole and len(samplers) == len(batch.items):
            nxt = self.scheduler.continue_decoding()
            if nxt is not None:
                try:
                    prepared = self.engine.prebuild(
                        [StepEntry(item.request.request_id, [0], [0]) for item in nxt.items])
                    if (self.run_ahead and cur.ids is not None
                            and all(r.sampling_params.repetition_penalty == 1.0 for r in samplers)
                            and len(nxt.items) == len(samplers)
                            and all(i.request is r for i, r in zip(nxt.items, samplers))):
                        logits = self.engine.run_prebuilt_fed(prepared, cur.ids, keep=False)
                        # the token that is still on its way counts for the sampler's counters
                        self._ahead = self._sample(nxt, samplers, logits, pending=1)
                    else:
                        self._early = (nxt, prepared)
                except Exception as exc:
                    # a step that could not be built or launched leaves nothing reserved; the
                    # step that is running is brought to its end first, then the error is raised
                    self._ahead = self._early = None
                    self.scheduler.abandon(nxt)
                    failed_ahead = exc
        sampled: dict[int, int] = {}
        if cur.ids is not None:
            cur.event.synchronize()
            host = cur.host.tolist()
            self.d2h_bytes_last = 4 * len(host)
            sampled = {r.request_id: int(host[k]) for r, k in zip(samplers, cur.rows)}
        self.steps_run += 1
        if self.steps_run % 256 == 0 and hasattr(self.engine.ops, "check_errors"):
            self.engine.ops.check_errors()
        done = self.scheduler.update(batch, sampled, advanced=True)
        if failed_ahead is not None:
            raise failed_ahead        # what finished in this step waits in `scheduler.finished`
        return done

    def _launch_next(self) -> "_Launched | None":
        """Schedule and launch a step (or launch the one prepared by the call before, if the
        state is still the one it was prepared for)."""
        early, self._early = self._early, None
        if early is not None and not (self.scheduler.still_valid(early[0])
                                      and self.engine.prebuilt_is_current(early[1])):
            self.scheduler.abandon(early[0])
            early = None
        if early is not None:
            batch, prepared = early
            samplers = [item.request for item in batch.items]
            try:
                logits = self.engine.run_prebuilt(prepared, [r.output_tokens[-1] for r in samplers],
                                                  keep=False)
            except Exception:
                self.scheduler.abandon(batch)
                raise
        else:
            batch = self.scheduler.schedule()
            if not batch.items:
                if self.scheduler.has_unfinished() and not batch.preempted:
                    raise RuntimeError("nothing can be scheduled: the cache is too small for the "
                                       "request at the head of the queue")
                return None
            entries = []
            samplers = []
            for item in batch.items:
                toks = item.request.tokens(item.start, item.num_tokens)
                entries.append(StepEntry(item.request.request_id, toks,
                                         [item.num_tokens - 1] if item.samples else []))
                if item.samples:
                    samplers.append(item.request)
            try:
                logits = self.engine.run_reserved(entries, keep=False)     # sampled from at once
            except Exception:
                # the requests stay where the scheduler put them, with nothing reserved: the
                # next call schedules them again
                self.scheduler.abandon(batch)
                raise
        try:
            return self._sample(batch, samplers, logits, pending=0)
        except Exception:
            self.scheduler.abandon(batch)
            raise

    def _sample(self, batch: ScheduledBatch, samplers: list[Request], logits: torch.Tensor,
                pending: int) -> "_Launched":
        """Launch the sampler on the step's logits and the copy of its ids to the host, into one
        of two pinned buffers in turn (the one of the step before may not have been read yet)."""
        if not samplers:
            return _Launched(batch, samplers, None, None, None, [], True)
        ids = self.sampler.sample(
            logits, [r.sampling_params for r in samplers],
            [len(r.output_tokens) + pending for r in samplers], [r.seed for r in samplers],
            [r.all_tokens if r.sampling_params.repetition_penalty != 1.0 else ()
             for r in samplers])
        n = len(samplers)
        self._ids_turn ^= 1
        turn = self._ids_turn
        if self._ids_host[turn] is None or self._ids_host[turn].numel() < n:
            self._ids_host[turn] = torch.empty(max(n, 64), dtype=torch.int32,
                                               pin_memory=self.device.type == "cuda")
            self._ids_event[turn] = (torch.cuda.Event() if self.device.type == "cuda"
                                     else _NoEvent())
        host = self._ids_host[turn][:n]
        host.copy_(ids, non_blocking=True)
        event = self._ids_event[turn]
        event.record()
        return _Launched(batch, samplers, ids, host, event, list(range(n)), True)

    def abort(self, request: Request) -> bool:
        """Stop a request between two steps; its pages go back at once.  A decode step that was
        launched ahead with a row for it drops that row; one that was only prepared is given
        back and scheduled again.  Returns whether the request was still unfinished."""
        return self.scheduler.abort(request)

    def run(self, requests: Sequence[tuple[int, Request]]) -> list[Request]:
        """Run until all `(arrival_step, request)` pairs are finished
        (somi_inference/core/continuous_batching.py:179-205)."""
        pending = deque(sorted(requests, key=lambda p: p[0]))
        finished: list[Request] = []
        step = 0
        while pending or self.scheduler.has_unfinished():
            while pending and pending[0][0] <= step:
                self.scheduler.add_request(pending.popleft()[1])
            finished.extend(self.step())
            self.scheduler.drain_finished()
            step += 1
        return finished

    # --------------------------------------------------------------- generate
    def generate(self, prompt: str | Sequence[int], *, max_new_tokens: int,
                 temperature: float = 1.0, top_k: int = -1, top_p: float = 1.0,
                 repetition_penalty: float = 1.0, seed: int | None = None,
                 ignore_eos: bool = False) -> str | list[int]:
        """Generate for one prompt; return only what is new (text for text, ids for ids)."""
        is_text = isinstance(prompt, str)
        tokens = self._tok().encode(prompt, add_special_tokens=False) if is_text else list(prompt)
        sp = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p,
                            repetition_penalty=repetition_penalty, seed=seed)
        req = self.make_request(tokens, max_new_tokens=max_new_tokens, sampling_params=sp,
                                ignore_eos=ignore_eos)
        finished = self.run([(0, req)])
        assert len(finished) == 1, "generate expects exactly one finished request"
        out = finished[0].output_tokens
        return self._tok().decode(out, skip_special_tokens=True) if is_text else out

    def generate_many(self, prompts: Sequence[Sequence[int]], *, max_new_tokens: int,
                      sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
                      arrival_steps: Sequence[int] | None = None,
                      ignore_eos: bool = False) -> list[list[int]]:
        """Several token-id prompts through the continuous-batching loop; outputs in input order."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        arrival_steps = arrival_steps or [0] * len(prompts)
        reqs = [self.make_request(p, max_new_tokens=max_new_tokens, sampling_params=sp,
                                  ignore_eos=ignore_eos)
                for p, sp in zip(prompts, sampling_params)]
        self.run(list(zip(arrival_steps, reqs)))
        return [r.output_tokens for r in reqs]

    def generate_stream(self, prompt: Sequence[int], *, max_new_tokens: int,
                        **sampling) -> Iterator[int]:
        """Yield new token ids one by one (the reference leaves streaming unimplemented,
        somi_inference/entrypoints/llm.py:166-170)."""
        sp = SamplingParams(**sampling)
        req = self.make_request(list(prompt), max_new_tokens=max_new_tokens, sampling_params=sp)
        self.scheduler.add_request(req)
        sent = 0
        try:
            while self.scheduler.has_unfinished():
                self.step()
                self.scheduler.drain_finished()
                while sent < len(req.output_tokens):
                    yield req.output_tokens[sent]
                    sent += 1
        finally:
            # a reader that stops early leaves nothing behind
            if self.abort(req):
                self.scheduler.drain_finished()
