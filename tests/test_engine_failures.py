"""Failure paths of the engine loop, on the CPU, with a stand-in for the step function: a step
that raises ends every live request with that error, gives every page and slot back, and leaves
the engine able to serve the next request (the reference's failure path:
v10_triton_paged_gqa/engine.py:204-217, scheduler.py:294-332)."""
import pytest

from torchlet_b200.cache import CacheManager, GroupSpec
from torchlet_b200.config import EngineConfig
from torchlet_b200.engine.engine import Engine
from torchlet_b200.engine.scheduler import Request, RequestState
from torchlet_b200.sampling import SamplingParams


class _Tokens(list):
    def tolist(self):
        return list(self)

    def numel(self):
        return len(self)


class _Result:
    def __init__(self, tokens):
        self.tokens = _Tokens(tokens) if tokens else None
        self.logits = None


class _Event:
    def synchronize(self):
        pass


class FailingRunner:
    """The runner's interface as the engine uses it.  'Samples' 1000 + the request's length;
    raises in the step numbered ``fail_at``."""

    def __init__(self, fail_at=None, num_pages=64, page=4, slots=3):
        self.cache = CacheManager([GroupSpec(1, 8, None, (0,), num_pages)], page, slots, 256)
        self.fail_at = fail_at
        self.steps_run = 0

    def admit(self, rid):
        return self.cache.admit(rid)

    def finish(self, rid):
        self.cache.finish(rid)

    def reserve(self, rid, new_len):
        return self.cache.extend(rid, new_len)

    def can_feed_previous(self, entries):
        return False

    def tokens_to_host(self, result):
        return result.tokens, _Event()

    def run(self, entries, feed_previous=False):
        if self.steps_run == self.fail_at:
            self.steps_run += 1
            raise RuntimeError("the step function failed")
        self.steps_run += 1
        tokens = []
        for e in entries:
            before = self.cache.num_tokens(e.request_id)
            assert self.cache.extend(e.request_id, before + len(e.tokens))
            self.cache.advance(e.request_id, before + len(e.tokens))
            if e.sample is not None:
                tokens.append(1000 + before + len(e.tokens))
        return _Result(tokens)


def _engine(runner):
    config = EngineConfig(max_decode_slots=3, kv_block_size=4, max_seq_len=256, max_num_batched_tokens=16, cuda_graph=False)
    return Engine(None, config, runner=runner)


def _requests():
    return [Request(list(range(n)), SamplingParams(max_new_tokens=5)) for n in (20, 3, 9, 30)]


@pytest.mark.parametrize("loop", ["run", "step"])
@pytest.mark.parametrize("fail_at", [0, 2, 5])
def test_a_failed_step_fails_every_request_and_the_engine_serves_again(loop, fail_at):
    runner = FailingRunner(fail_at=fail_at)
    engine = _engine(runner)
    requests = _requests()
    engine.add_requests(requests)
    with pytest.raises(RuntimeError, match="step function failed"):
        if loop == "run":
            engine.run()
        else:
            while engine.scheduler.has_work():
                engine.step()
    # every request that had not finished ends with the error; nothing is held any more
    assert all(r.state is RequestState.FINISHED for r in requests)
    unfinished = [r for r in requests if len(r.output_tokens) < 5]
    assert unfinished and all(isinstance(r.error, RuntimeError) for r in unfinished)
    assert not engine.scheduler.has_work() and engine.scheduler.drain_finished() == []
    runner.cache.check()
    assert runner.cache.live_requests() == [] and runner.cache.num_free_slots == 3
    assert runner.cache.pools[0].num_free == runner.cache.pools[0].num_pages - 1
    # a fresh request is served afterwards
    fresh = Request(list(range(11)), SamplingParams(max_new_tokens=4))
    engine.generate([fresh])
    assert fresh.error is None and fresh.output_tokens == [1011, 1012, 1013, 1014]
    runner.cache.check()


@pytest.mark.parametrize("loop", ["run", "step"])
def test_an_interrupt_from_the_keyboard_leaves_nothing_half_run(loop):
    class Interrupted(FailingRunner):
        def run(self, entries, feed_previous=False):
            if self.steps_run == 3:
                self.steps_run += 1
                raise KeyboardInterrupt
            return super().run(entries, feed_previous)

    runner = Interrupted()
    engine = _engine(runner)
    requests = _requests()
    engine.add_requests(requests)
    with pytest.raises(KeyboardInterrupt):
        if loop == "run":
            engine.run()
        else:
            while engine.scheduler.has_work():
                engine.step()
    assert all(r.state is RequestState.FINISHED for r in requests) and not engine.scheduler.has_work()
    assert any(isinstance(r.error, KeyboardInterrupt) for r in requests)
    runner.cache.check()
    assert runner.cache.live_requests() == [] and runner.cache.num_free_slots == 3
    fresh = Request(list(range(11)), SamplingParams(max_new_tokens=4))
    engine.generate([fresh])
    assert fresh.error is None and fresh.output_tokens == [1011, 1012, 1013, 1014]


def test_without_a_failure_both_loops_agree():
    outputs = []
    for loop in ("run", "step"):
        engine = _engine(FailingRunner())
        requests = _requests()
        engine.add_requests(requests)
        if loop == "run":
            engine.run()
        else:
            while engine.scheduler.has_work():
                engine.step()
        assert all(r.error is None for r in requests)
        outputs.append([r.output_tokens for r in requests])
    assert outputs[0] == outputs[1]


def test_the_loop_serves_requests_that_arrive_while_others_run():
    """``Engine.run(poll)``: requests handed in by the poll callable between steps are admitted in
    order of arrival; the loop ends when the source is exhausted and everything is finished."""
    engine = _engine(FailingRunner())
    requests = _requests() + [Request(list(range(6)), SamplingParams(max_new_tokens=3))]
    schedule = {0: requests[:1], 3: requests[1:3], 4: [], 9: requests[3:]}
    calls = [0]

    def poll():
        turn = calls[0]
        calls[0] += 1
        if turn > 9:
            return None
        return schedule.get(turn, [])

    ended = engine.run(poll)
    assert calls[0] >= 11 and {id(r) for r in ended} == {id(r) for r in requests}
    assert all(r.error is None and r.state is RequestState.FINISHED for r in requests)
    assert [r.output_tokens for r in requests][-1] == [1006, 1007, 1008]
    assert engine.runner.cache.live_requests() == []
    # an idle loop keeps asking until the source says that nothing more will come
    idle = _engine(FailingRunner())
    late = Request(list(range(4)), SamplingParams(max_new_tokens=2))
    answers = iter([[], [], [late], [], None])
    idle.run(lambda: next(answers))
    assert late.output_tokens == [1004, 1005]


# ------------------------------------------------------------- the loop as an asyncio task
def _expected(prompt_len, new_tokens):
    return [1000 + prompt_len + k for k in range(new_tokens)]


def test_coroutines_hand_in_requests_while_the_loop_runs():
    """The reference's manner of use (v10_triton_paged_gqa/llm.py:113-140): several coroutines
    that start at different times await their requests; one loop, an asyncio task, serves them
    all, and ``shutdown`` ends it."""
    import asyncio

    engine = _engine(FailingRunner())

    async def caller(delay, lengths, new_tokens):
        await asyncio.sleep(delay)
        requests = [Request(list(range(n)), SamplingParams(max_new_tokens=new_tokens)) for n in lengths]
        assert await engine.submit(requests) is requests
        return requests

    async def main():
        try:
            groups = await asyncio.gather(caller(0.0, (20, 3), 6), caller(0.01, (9,), 4), caller(0.02, (30, 5, 7), 3))
            task = engine._task
            assert task is not None and not task.done()  # the loop idles, it has not ended
            late = await caller(0.0, (11,), 2)  # ... and serves a later caller with the same task
            assert engine._task is task
            return groups + [late]
        finally:
            await engine.shutdown()

    groups = asyncio.run(main())
    for group in groups:
        for request in group:
            assert request.error is None and request.state is RequestState.FINISHED
            assert request.output_tokens == _expected(len(request.prompt_tokens), request.params.max_new_tokens)
    assert engine._task is None and not engine._waiting_callers and not engine._inbox
    engine.runner.cache.check()
    assert engine.runner.cache.live_requests() == [] and engine.runner.cache.num_free_slots == 3


def test_shutdown_ends_live_requests_and_the_engine_starts_again():
    import asyncio

    engine = _engine(FailingRunner())
    long = [Request(list(range(n)), SamplingParams(max_new_tokens=200)) for n in (20, 9, 4, 6)]

    async def main():
        waiting = asyncio.create_task(engine.submit(long))
        for _ in range(50):  # let the loop run some steps
            await asyncio.sleep(0)
        assert any(r.output_tokens for r in long) and not waiting.done()
        await engine.shutdown()
        assert (await waiting) is long  # the caller is released, its requests carry the reason
        fresh = [Request(list(range(11)), SamplingParams(max_new_tokens=4))]
        await engine.submit(fresh)  # a new task serves the next caller
        await engine.shutdown()
        return fresh

    fresh = asyncio.run(main())
    import asyncio as _a
    assert all(isinstance(r.error, _a.CancelledError) and r.state is RequestState.FINISHED for r in long)
    assert fresh[0].error is None and fresh[0].output_tokens == _expected(11, 4)
    engine.runner.cache.check()
    assert engine.runner.cache.live_requests() == [] and engine.runner.cache.num_free_slots == 3
    assert engine.runner.cache.pools[0].num_free == engine.runner.cache.pools[0].num_pages - 1


def test_a_failed_step_releases_every_waiting_coroutine():
    import asyncio

    engine = _engine(FailingRunner(fail_at=3))

    async def main():
        first = [Request(list(range(n)), SamplingParams(max_new_tokens=8)) for n in (20, 3)]
        second = [Request(list(range(9)), SamplingParams(max_new_tokens=8))]
        await asyncio.gather(engine.submit(first), engine.submit(second))
        assert engine._task.done()  # the loop ended with the failure ...
        third = [Request(list(range(5)), SamplingParams(max_new_tokens=3))]
        await engine.submit(third)  # ... and the next caller gets a new one
        await engine.shutdown()
        return first + second, third

    failed, third = asyncio.run(main())
    assert all(r.state is RequestState.FINISHED for r in failed)
    assert any(isinstance(r.error, RuntimeError) for r in failed)
    assert all(isinstance(r.error, RuntimeError) or len(r.output_tokens) == 8 for r in failed)
    assert third[0].error is None and third[0].output_tokens == _expected(5, 3)
    engine.runner.cache.check()
    assert engine.runner.cache.live_requests() == []


def test_submit_refuses_a_bad_request_before_anything_is_handed_in():
    import asyncio

    engine = _engine(FailingRunner())

    async def main():
        good = Request(list(range(5)), SamplingParams(max_new_tokens=2))
        with pytest.raises(ValueError):
            await engine.submit([good, Request([], SamplingParams(max_new_tokens=2))])
        assert not engine._inbox and not engine._waiting_callers and good.state is RequestState.WAITING
        await engine.shutdown()

    asyncio.run(main())
