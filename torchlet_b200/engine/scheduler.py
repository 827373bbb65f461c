"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

Request states and the waiting/running/finished lists are the reference's
(v10_triton_paged_gqa/request.py:7-24, scheduler.py:41-43), so are admission in
arrival order while a slot is free (scheduler.py:132-155), the validation of a
request's length (scheduler.py:84-95) and the finishing rules (scheduler.py:255-266:
a sampled stop id ends the request and is not emitted; ``max_new_tokens`` outputs end
it).  Different from the reference:

* one mixed batch per step instead of a prefill forward and a decode forward;
* a token budget: decoding requests take one token each first, what is left goes to
  portions of prompts, which may be cut anywhere;
* when pages run out, the request admitted LAST is preempted: its pages and slot are
  given back, it returns to the front of the waiting list and is later recomputed from
  its prompt plus the tokens it has produced (the reference keeps the pages and loses
  the request, scheduler.py:106-109, 134-143).  A request that cannot get pages even
  when it runs alone fails by itself with an error; the others go on.

The scheduler is host-only: it talks to a ``runner`` object that offers
``admit(id)``, ``finish(id)``, ``reserve(id, new_len) -> bool`` and ``cache``
(a ``CacheManager``), so it is tested on the CPU with a stand-in runner.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from enum import Enum
from typing import Optional

from ..cache.manager import CacheError
from ..sampling import SampleSpec, SamplingParams


class RequestState(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


_arrival = itertools.count()


@dataclass(eq=False)  # requests compare by identity (and list searches stay cheap)
class Request:
    prompt_tokens: list
    params: SamplingParams = field(default_factory=SamplingParams)
    request_id: Optional[str] = None
    output_tokens: list = field(default_factory=list)
    state: RequestState = RequestState.WAITING
    error: Optional[Exception] = None
    num_computed: int = 0  # tokens whose keys and values are in the cache
    preemptions: int = 0
    arrival: int = field(default_factory=lambda: next(_arrival))
    prompt: str = ""
    output: str = ""

    def __post_init__(self) -> None:
        if self.request_id is None:
            self.request_id = f"req-{self.arrival}"
        self.prompt_tokens = [int(t) for t in self.prompt_tokens]

    @property
    def all_tokens(self) -> list:
        return self.prompt_tokens + self.output_tokens

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_tokens) + len(self.output_tokens)

    @property
    def seed(self) -> int:
        return self.params.seed if self.params.seed is not None else 0x5EED0000 + self.arrival


@dataclass
class ScheduledPortion:
    request: Request
    start: int  # first token of the portion within request.all_tokens
    length: int
    samples: bool  # the portion reaches the request's last known token: sample the next one


@dataclass
class StepPlan:
    portions: list
    preempted: list
    failed: list

    @property
    def num_tokens(self) -> int:
        return sum(p.length for p in self.portions)


@dataclass
class SchedulerStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    failed: int = 0
    finished: int = 0
    peak_running: int = 0
    peak_pages: int = 0  # the most pages held at once, over all pools


class Scheduler:
    def __init__(self, runner, max_num_batched_tokens: int, max_seq_len: int, admission_headroom=1):
        """``admission_headroom``: see ``_room_to_admit`` (None: admit on the first portion's pages)."""
        if max_num_batched_tokens <= 0:
            raise ValueError("max_num_batched_tokens must be positive")
        if admission_headroom is not None and admission_headroom < 0:
            raise ValueError("admission_headroom must be None or at least 0")
        self.admission_headroom = admission_headroom
        self.runner = runner
        self.cache = runner.cache
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_seq_len = max_seq_len
        self.waiting: list[Request] = []
        self.running: list[Request] = []  # in admission order
        self.finished: list[Request] = []
        self.stats = SchedulerStats()

    # -------------------------------------------------------------- requests
    def validate(self, request: Request) -> None:
        if request.params.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        if not request.prompt_tokens:
            raise ValueError("a request needs at least one prompt token")
        needed = len(request.prompt_tokens) + request.params.max_new_tokens - 1
        if needed > self.max_seq_len:
            raise ValueError(
                f"request {request.request_id} requires {needed} cache positions, "
                f"but max_seq_len is {self.max_seq_len}"
            )

    def add_request(self, request: Request) -> None:
        self.validate(request)
        request.state = RequestState.WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -------------------------------------------------------------- schedule
    def _preempt(self, request: Request) -> None:
        self.runner.finish(request.request_id)
        self.running.remove(request)
        request.state = RequestState.WAITING
        request.num_computed = 0
        request.preemptions += 1
        self.waiting.insert(0, request)
        self.stats.preemptions += 1

    def _fail(self, request: Request, error: Exception) -> None:
        if self.cache.has(request.request_id):
            self.runner.finish(request.request_id)
        if request in self.running:
            self.running.remove(request)
        if request in self.waiting:
            self.waiting.remove(request)
        request.state = RequestState.FINISHED
        request.error = error
        self.finished.append(request)
        self.stats.failed += 1

    def _reserve(self, request: Request, length: int, scheduled: dict, plan: StepPlan) -> int:
        """Pages for ``length`` more tokens of ``request``, preempting later-admitted
        requests while needed.  Returns the length reserved (0: not this step)."""
        while True:
            if self.runner.reserve(request.request_id, request.num_computed + length):
                return length
            victim = self.running[-1]
            if victim is request:
                others_hold_pages = len(self.running) > 1
                if others_hold_pages or scheduled:
                    # wait for earlier requests to finish; give this one's pages back meanwhile
                    self._preempt(request)
                    plan.preempted.append(request)
                else:
                    self._fail(request, CacheError(
                        f"request {request.request_id} cannot get cache pages for "
                        f"{request.num_computed + length} tokens even alone: the page pool is too small"))
                    plan.failed.append(request)
                return 0
            scheduled.pop(victim.request_id, None)
            self._preempt(victim)
            plan.preempted.append(victim)

    def _room_to_admit(self, request: Request) -> bool:
        """Whether the pools have room to take ``request`` in beside the running ones: pages for
        all the tokens it has (the reference admits on the whole prompt too,
        v10_triton_paged_gqa/scheduler.py:132-155) and ``admission_headroom`` pages for every
        running request to grow into.  Without the rule a request is admitted on the pages of its
        first portion alone, and under a tight pool the last admitted ones are preempted again and
        again (measured at Qwen2.5-0.5B sizes, 1,024 requests: 454 preemptions and 223 k recomputed
        tokens against 45 and 22 k with a headroom of one page, output tokens a second +3 %).
        With nothing running a request is always admitted: whether it fits at all shows when it runs.
        (Every group is asked for the pages of all the tokens, a windowed one too, which will hold
        fewer at a time: the rule errs on the side of waiting.)"""
        if self.admission_headroom is None or not self.running:
            return True
        pages = -(-request.num_tokens // self.cache.page_size)
        reserve = self.admission_headroom * len(self.running)
        return all(pool.num_free >= pages + reserve for pool in self.cache.pools)

    def schedule(self) -> StepPlan:
        """Decide the next step: which requests run how many of their tokens."""
        plan = StepPlan([], [], [])
        budget = self.max_num_batched_tokens
        scheduled: dict = {}  # request_id -> ScheduledPortion, in order

        # 1. decoding requests first, one token each (oldest first)
        prompts_left = False
        for request in list(self.running):
            if budget <= 0:
                break
            if request.state is not RequestState.RUNNING:  # preempted earlier in this loop
                continue
            if len(request.prompt_tokens) + len(request.output_tokens) - request.num_computed != 1:
                prompts_left = True
                continue
            if self._reserve(request, 1, scheduled, plan):
                scheduled[request.request_id] = ScheduledPortion(request, request.num_computed, 1, True)
                budget -= 1

        # 2. portions of requests that are still reading their prompt (or being recomputed)
        for request in (list(self.running) if prompts_left else ()):
            if request.state is not RequestState.RUNNING or budget <= 0 or request.request_id in scheduled:
                continue
            remaining = request.num_tokens - request.num_computed
            length = min(remaining, budget)
            if length > 0 and self._reserve(request, length, scheduled, plan):
                scheduled[request.request_id] = ScheduledPortion(
                    request, request.num_computed, length, length == remaining)
                budget -= length

        # 3. admit waiting requests in order while slots, pages and budget last
        while self.waiting and budget > 0 and self.cache.num_free_slots > 0:
            request = self.waiting[0]
            if plan.preempted and request in plan.preempted:
                break  # preempted in this very step: wait for pages
            length = min(request.num_tokens, budget)
            if not self._room_to_admit(request):
                break
            self.runner.admit(request.request_id)
            if not self.runner.reserve(request.request_id, length):
                self.runner.finish(request.request_id)
                if not self.running and not scheduled:
                    self.waiting.pop(0)
                    self._fail(request, CacheError(
                        f"request {request.request_id} cannot get cache pages for {length} tokens "
                        "even alone: the page pool is too small"))
                    plan.failed.append(request)
                    continue
                break
            self.waiting.pop(0)
            request.state = RequestState.RUNNING
            request.num_computed = 0
            self.running.append(request)
            scheduled[request.request_id] = ScheduledPortion(request, 0, length, length == request.num_tokens)
            budget -= length

        plan.portions = list(scheduled.values())
        self.stats.peak_running = max(self.stats.peak_running, len(self.running))
        self.stats.peak_pages = sum(pool.peak_held for pool in self.cache.pools)
        return plan

    # ---------------------------------------------------------------- update
    def sample_spec(self, request: Request) -> SampleSpec:
        return SampleSpec(request.params.temperature, request.seed, len(request.output_tokens))

    def update(self, plan: StepPlan, sampled_tokens: list) -> list:
        """Apply a step's result: advance every portion's request, append the sampled
        tokens (in the order of the sampling portions), finish and free.  Returns the
        requests that finished in this step."""
        done = []
        sampled = iter(sampled_tokens)
        self.stats.steps += 1
        for portion in plan.portions:
            request = portion.request
            request.num_computed += portion.length
            if portion.length == 1 and portion.start >= len(request.prompt_tokens):
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += portion.length
            if not portion.samples:
                continue
            token = int(next(sampled))
            params = request.params
            if not params.ignore_eos and token in params.stop_token_ids:
                finished = True
            else:
                request.output_tokens.append(token)
                finished = len(request.output_tokens) >= params.max_new_tokens
            if finished:
                request.state = RequestState.FINISHED
                self.running.remove(request)
                self.runner.finish(request.request_id)
                self.finished.append(request)
                self.stats.finished += 1
                done.append(request)
        return done

    def fail_all(self, error: Exception) -> list:
        """Every waiting or running request ends with ``error``; everything held is
        given back (the reference's failure path, scheduler.py:294-332)."""
        failed = []
        for request in self.running + self.waiting:
            if self.cache.has(request.request_id):
                self.runner.finish(request.request_id)
            request.state = RequestState.FINISHED
            request.error = error
            failed.append(request)
        self.running, self.waiting = [], []
        self.finished.extend(failed)
        self.stats.failed += len(failed)
        return failed

    def drain_finished(self) -> list:
        finished, self.finished = self.finished, []
        return finished
