"""The engine: scheduler above, step function below, one loop.

One ``step()`` = schedule -> run the mixed batch -> sample -> apply tokens -> free what
finished (the reference's loop: v10_triton_paged_gqa/engine.py:101-135, 204-217).
``step()`` is synchronous; ``run()`` keeps one decode step ahead of the tokens it has seen
(see ``_next_decode``).  A failure inside a step ends every live request with that error
and gives all pages and slots back, as the reference's ``fail_all`` does
(engine.py:215-217).

The reference is used from coroutines: its loop is an asyncio task that ``start()`` creates,
callers ``await`` their requests while it runs, ``shutdown()`` cancels it
(engine.py:77-99, llm.py:84-110).  ``start`` / ``submit`` / ``shutdown`` here do the same around
the very loop that ``run`` drives: between two iterations the task yields to the other
coroutines, which is when they hand in requests.
"""
from __future__ import annotations

import asyncio
from typing import Optional

from .. import ops
from ..config.engine import EngineConfig
from ..logger import logger
from ..parts.model import LayeredModel
from ..sampling import SampleSpec
from .runner import ModelRunner, OutOfPages, StepEntry
from .scheduler import Request, RequestState, ScheduledPortion, Scheduler, StepPlan


class Engine:
    def __init__(self, model: LayeredModel, config: Optional[EngineConfig] = None, runner=None):
        """``runner``: the step function to drive, default a ``ModelRunner`` over ``model`` (tests
        of the loop's own decisions pass a stand-in and no model)."""
        self.config = config or EngineConfig()
        self.runner = runner if runner is not None else ModelRunner(model, self.config)
        self.scheduler = Scheduler(self.runner, self.config.max_num_batched_tokens, self.config.max_seq_len,
                                   self.config.admission_headroom)
        self.steps_ahead = 0  # decode steps launched before the tokens of the step before were read
        # the loop as an asyncio task: requests handed in and not yet seen by the loop, who waits for which
        self._task = None
        self._inbox: list = []
        self._waiting_callers: dict = {}
        self._wake = None

    def add_requests(self, requests: list) -> None:
        for request in requests:
            self.scheduler.validate(request)
        for request in requests:
            self.scheduler.add_request(request)

    def _entries(self, plan) -> list:
        scheduler = self.scheduler
        entries = []
        for portion in plan.portions:
            request = portion.request
            prompt_len = len(request.prompt_tokens)
            if portion.start >= prompt_len:  # decoding (or recomputing produced tokens)
                first = portion.start - prompt_len
                tokens = request.output_tokens[first:first + portion.length]
            elif portion.start + portion.length <= prompt_len:
                tokens = request.prompt_tokens[portion.start:portion.start + portion.length]
            else:
                tokens = request.all_tokens[portion.start:portion.start + portion.length]
            entries.append(StepEntry(request.request_id, tokens,
                                     sample=scheduler.sample_spec(request) if portion.samples else None))
        return entries

    def step(self) -> list:
        """One engine step; returns the requests that finished (or failed) in it.  A failure
        inside the step ends every live request with that error, gives everything back, and
        is raised again."""
        scheduler = self.scheduler
        try:
            plan = scheduler.schedule()
            done = list(plan.failed)
            if plan.portions:
                result = self.runner.run(self._entries(plan))
                sampled = result.tokens.tolist() if result.tokens is not None else []
                done += scheduler.update(plan, sampled)
                if done:  # nothing is handed back before the kernels' own error words have been read
                    self._check_kernels(done)
        except BaseException as exc:  # also an interrupt from the keyboard: nothing stays half-run
            self._fail_everything(exc)
            raise
        scheduler.drain_finished()
        return done

    @staticmethod
    def _check_kernels(done: list) -> None:
        """Raises if a kernel has given up a bounded wait since the last check; the requests that
        have just finished did so on tokens of such a step and end with that error as well."""
        try:
            ops.raise_on_wait_errors()
        except Exception as exc:
            for request in done:
                if request.error is None:
                    request.error = exc
            raise

    def _fail_everything(self, exc: Exception) -> list:
        """A failed step fails every live request (the reference: engine.py:215-217)."""
        logger.error("engine step failed: %s", exc)
        failed = self.scheduler.fail_all(exc)
        self.scheduler.drain_finished()
        return failed

    # ----------------------------------------------------- decode, one step ahead
    # While every running request decodes, the next step's inputs are known before this
    # step's tokens are: positions and pages follow from the lengths, and the token itself
    # can be handed over on the device.  ``run`` therefore launches step k + 1 before it
    # reads step k's tokens, so that the host's share of a step (scheduling, metadata, the
    # copy of the tokens) runs beside the GPU and not between two of its steps.  A request
    # that ends at step k for a reason the host could not foresee (a stop token) has run one
    # step too many by then; its lane of step k + 1 is dropped, and its pages, given back
    # at step k, are reused only by steps launched later on the same stream.
    def _next_decode(self, plan):
        """The plan and entries of the step after ``plan`` if that can be told without its
        tokens: every running request is in ``plan`` with one decoded token and stays under
        its token limit, and nothing waits for a free slot.  Else None."""
        scheduler = self.scheduler
        if not self.config.cuda_graph or len(plan.portions) != len(scheduler.running):
            return None
        if scheduler.waiting and self.runner.cache.num_free_slots > 0:
            return None
        portions, entries = [], []
        for portion in plan.portions:
            request = portion.request
            produced = len(request.output_tokens)
            if (portion.length != 1 or not portion.samples or portion.start < len(request.prompt_tokens)
                    or produced + 2 > request.params.max_new_tokens
                    or request.num_tokens + 2 > self.runner.cache.max_seq_len):
                return None
            portions.append(ScheduledPortion(request, portion.start + 1, 1, True))
            entries.append(StepEntry(request.request_id, [0],
                                     sample=SampleSpec(request.params.temperature, request.seed, produced + 1)))
        if not self.runner.can_feed_previous(entries):
            return None
        return StepPlan(portions, [], []), entries

    IDLE = object()  # what the loop yields when it has nothing to do and its source nothing to give

    def run(self, poll=None) -> list:
        """Step until no request is waiting or running; returns all that ended.

        ``poll``: a callable asked before every scheduling decision for the requests that have
        arrived since the last call (a list, possibly empty), as the reference's loop drains its
        queue every iteration (v10_triton_paged_gqa/scheduler.py:122-128); it returns None once
        no more will come.  With it the loop serves requests that arrive while others run.  While
        nothing is running ``poll`` is asked again at once: a source that has nothing yet should
        wait inside its own call (the asyncio task of ``start`` waits for an event instead)."""
        ended = []
        for chunk in self._loop(poll):
            if chunk is not Engine.IDLE:
                ended += chunk
        return ended

    def _loop(self, poll):
        """The loop itself, as a generator: after every iteration it yields the requests that
        ended in it (``IDLE`` when there was nothing to do), so that its driver may do something
        between two iterations.  A failed step fails every live request and is raised."""
        scheduler, runner = self.scheduler, self.runner
        ahead = None  # (plan, pinned tokens, event) of a step that is launched but not yet applied
        try:
            while ahead is not None or scheduler.has_work() or poll is not None:
                ended = []
                if poll is not None:
                    arrived = poll()
                    if arrived is None:
                        poll = None
                    elif arrived:
                        self.add_requests(arrived)
                    if ahead is None and not scheduler.has_work():
                        if poll is not None:
                            yield Engine.IDLE
                        continue
                if ahead is None:
                    plan = scheduler.schedule()
                    ended += plan.failed
                    if not plan.portions:
                        scheduler.drain_finished()
                        yield ended
                        continue
                    result = runner.run(self._entries(plan))
                    if result.tokens is None:  # portions of prompts that sample nothing
                        scheduler.update(plan, [])
                        scheduler.drain_finished()
                        yield ended
                        continue
                    ahead = (plan, *runner.tokens_to_host(result))
                plan, tokens, event = ahead
                ahead = None
                following = self._next_decode(plan)
                if following is not None:
                    try:
                        result = runner.run(following[1], feed_previous=True)
                        ahead = (following[0], *runner.tokens_to_host(result))
                        self.steps_ahead += 1
                    except OutOfPages:  # the scheduler decides who gives way, with this step's tokens in hand
                        ahead = None
                event.synchronize()
                values = tokens.tolist()
                if any(p.request.state is not RequestState.RUNNING for p in plan.portions):
                    # lanes of requests that ended one step earlier: that step was launched before the host knew
                    live = [(p, v) for p, v in zip(plan.portions, values) if p.request.state is RequestState.RUNNING]
                    plan = StepPlan([p for p, _ in live], [], [])
                    values = [v for _, v in live]
                done = scheduler.update(plan, values)
                if done:
                    self._check_kernels(done)  # nothing is handed back before the kernels' error words are read
                    ended += done
                scheduler.drain_finished()
                yield ended
        except GeneratorExit:  # the driver stops the loop between two iterations (shutdown): its business
            raise
        except BaseException as exc:  # a failed step (or an interrupt from the keyboard) fails every live request
            self._fail_everything(exc)
            raise

    def generate(self, requests: list) -> list:
        self.add_requests(requests)
        self.run()
        return requests

    # ------------------------------------------------------------ the loop as an asyncio task
    def start(self) -> None:
        """Start the loop as a task of the running event loop unless it is running already
        (the reference: engine.py:77-79)."""
        if self._task is None or self._task.done():
            self._wake = asyncio.Event()
            self._task = asyncio.get_running_loop().create_task(self._serve())

    async def submit(self, requests: list) -> list:
        """Hand requests to the running loop (started if need be) and wait until every one of
        them has ended; returns them (``error`` set on those that failed).  Several coroutines
        may wait at the same time: their requests share the loop's batches."""
        for request in requests:
            self.scheduler.validate(request)
        self.start()
        loop = asyncio.get_running_loop()
        futures = []
        for request in requests:
            futures.append(loop.create_future())
            self._waiting_callers[request] = futures[-1]
        self._inbox.extend(requests)
        self._wake.set()
        await asyncio.gather(*futures)
        return requests

    async def shutdown(self) -> None:
        """Cancel the loop; whatever is live or handed in ends with ``asyncio.CancelledError`` as
        its error, and every page and slot comes back (the reference: engine.py:81-96)."""
        task, self._task = self._task, None
        if task is None:
            return
        if not task.done():
            task.cancel()
            try:
                await task
            except asyncio.CancelledError:
                pass
        self._end_everything(asyncio.CancelledError())

    def _end_everything(self, exc: BaseException) -> None:
        """After the loop has stopped: what the scheduler still holds and what it never saw ends
        with ``exc``; every waiting caller is released."""
        self.scheduler.fail_all(exc)
        self.scheduler.drain_finished()
        for request in self._inbox:
            request.error, request.state = exc, RequestState.FINISHED
        self._inbox = []
        self._release(list(self._waiting_callers))

    def _release(self, requests: list) -> None:
        for request in requests:
            future = self._waiting_callers.pop(request, None)
            if future is not None and not future.done():
                future.set_result(request)

    async def _serve(self) -> None:
        def poll():
            arrived, self._inbox = self._inbox, []
            return arrived  # never None: the task lives until it is cancelled

        loop = self._loop(poll)
        try:
            for ended in loop:
                if ended is Engine.IDLE:
                    self._wake.clear()
                    if not self._inbox:
                        await self._wake.wait()
                    continue
                self._release(ended)
                await asyncio.sleep(0)  # the other coroutines' turn: this is when requests arrive
        except asyncio.CancelledError:
            loop.close()
            raise
        except Exception as exc:  # the loop has failed everything it held; the task ends, start() makes a new one
            self._end_everything(exc)

