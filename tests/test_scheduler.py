"""The scheduler's decisions, on the CPU, with a stand-in for the step function."""
import random

import pytest

from torchlet_b200.cache import CacheManager, GroupSpec
from torchlet_b200.engine.scheduler import Request, RequestState, Scheduler
from torchlet_b200.sampling import SamplingParams


class FakeRunner:
    """Offers what the scheduler needs of a runner; 'samples' token = position count."""

    def __init__(self, num_pages=64, page=4, slots=4, max_seq=256, window=None):
        self.cache = CacheManager([GroupSpec(1, 8, window, (0,), num_pages)], page, slots, max_seq)

    def admit(self, rid):
        return self.cache.admit(rid)

    def finish(self, rid):
        self.cache.finish(rid)

    def reserve(self, rid, new_len):
        return self.cache.extend(rid, new_len)

    def run(self, plan):
        tokens = []
        for portion in plan.portions:
            rid = portion.request.request_id
            assert self.cache.num_tokens(rid) == portion.start, "a portion must continue where the cache ends"
            self.cache.advance(rid, portion.start + portion.length)
            if portion.samples:
                tokens.append(1000 + portion.start + portion.length)
        return tokens


def drive(sched, runner, max_steps=10_000):
    plans = []
    while sched.has_work():
        plan = sched.schedule()
        plans.append(plan)
        sched.update(plan, runner.run(plan))
        runner.cache.check()
        assert len(plans) < max_steps
    return plans


def req(n, new=4, **kw):
    return Request(list(range(n)), SamplingParams(max_new_tokens=new, **kw))


def test_budget_cuts_prompts_and_decodes_first():
    runner = FakeRunner()
    sched = Scheduler(runner, max_num_batched_tokens=10, max_seq_len=256)
    a, b = req(23, new=3), req(5, new=3)
    sched.add_request(a); sched.add_request(b)
    p1 = sched.schedule()
    assert [(p.request is a, p.start, p.length, p.samples) for p in p1.portions] == [(True, 0, 10, False)]
    sched.update(p1, runner.run(p1))
    p2 = sched.schedule(); sched.update(p2, runner.run(p2))
    assert [(p.start, p.length) for p in p2.portions] == [(10, 10)]
    p3 = sched.schedule()  # a's last 3 prompt tokens (sampling) beside b's whole prompt
    assert [(p.request is a, p.start, p.length, p.samples) for p in p3.portions] == [(True, 20, 3, True), (False, 0, 5, True)]
    sched.update(p3, runner.run(p3))
    p4 = sched.schedule()  # both decode: one token each
    assert [(p.length, p.samples) for p in p4.portions] == [(1, True), (1, True)]
    assert p4.portions[0].start == 23 and a.output_tokens == [1023]


def test_finishing_rules_and_everything_is_given_back():
    runner = FakeRunner()
    sched = Scheduler(runner, 64, 256)
    a = req(6, new=3)
    b = Request(list(range(4)), SamplingParams(max_new_tokens=10, stop_token_ids=(1006,)))  # third sampled token
    c = Request(list(range(4)), SamplingParams(max_new_tokens=4, stop_token_ids=(1005,), ignore_eos=True))
    for r in (a, b, c):
        sched.add_request(r)
    drive(sched, runner)
    assert a.output_tokens == [1006, 1007, 1008] and a.state is RequestState.FINISHED
    assert b.output_tokens == [1004, 1005]  # the stop token is not emitted
    assert c.output_tokens == [1004, 1005, 1006, 1007]
    assert runner.cache.live_requests() == [] and runner.cache.pools[0].num_free == 63
    assert sched.stats.finished == 3 and sched.stats.decode_tokens == 2 + 2 + 3


def test_validation():
    sched = Scheduler(FakeRunner(max_seq=16), 64, 16)
    with pytest.raises(ValueError, match="cache positions"):
        sched.add_request(req(10, new=8))
    sched.add_request(req(10, new=7))
    with pytest.raises(ValueError):
        sched.add_request(req(0))
    with pytest.raises(ValueError):
        sched.add_request(req(3, new=0))


def test_more_requests_than_slots_wait_in_order():
    runner = FakeRunner(slots=2)
    sched = Scheduler(runner, 64, 256)
    reqs = [req(5, new=2) for _ in range(5)]
    for r in reqs:
        sched.add_request(r)
    order = []
    while sched.has_work():
        plan = sched.schedule()
        assert len(sched.running) <= 2
        for r in sched.update(plan, runner.run(plan)):
            order.append(reqs.index(r))
    assert order == [0, 1, 2, 3, 4]


def test_pages_run_out_latest_is_preempted_and_recomputed():
    # 6 usable pages of 4 tokens; two requests of 9 prompt tokens (3 pages each) then decode
    # (admitted on the pages of their prompts alone: the admission rule below would make b wait)
    runner = FakeRunner(num_pages=7, page=4, slots=4)
    sched = Scheduler(runner, 64, 256, admission_headroom=None)
    a, b = req(9, new=8), req(9, new=8)
    sched.add_request(a); sched.add_request(b)
    plans = drive(sched, runner)
    assert any(b in p.preempted for p in plans) and not any(a in p.preempted for p in plans)
    assert b.preemptions >= 1 and a.preemptions == 0
    assert a.error is None and b.error is None
    assert len(a.output_tokens) == 8 and len(b.output_tokens) == 8
    # outputs do not depend on preemption: token = 1000 + position
    assert a.output_tokens == [1009 + i for i in range(8)] and b.output_tokens == a.output_tokens
    assert runner.cache.pools[0].num_free == 6 and sched.stats.preemptions >= 1


def test_admission_leaves_the_running_requests_room_to_grow():
    """The same two requests under the admission rule (pages for all of a request's tokens and
    one page of headroom for every running request): b waits until a has finished, nobody is
    preempted, the outputs are the same.  With room enough both run together from the start."""
    runner = FakeRunner(num_pages=7, page=4, slots=4)
    sched = Scheduler(runner, 64, 256)  # admission_headroom=1
    a, b = req(9, new=8), req(9, new=8)
    sched.add_request(a); sched.add_request(b)
    plans = drive(sched, runner)
    assert not any(p.preempted for p in plans) and sched.stats.preemptions == 0
    assert all(len(p.portions) == 1 for p in plans), "b ran beside a although the pool had no room for both to grow"
    assert a.output_tokens == [1009 + i for i in range(8)] and b.output_tokens == a.output_tokens
    assert runner.cache.pools[0].num_free == 6
    roomy = FakeRunner(num_pages=12, page=4, slots=4)  # 11 usable pages: 3 + 3 and headroom
    sched = Scheduler(roomy, 64, 256)
    a, b = req(9, new=8), req(9, new=8)
    sched.add_request(a); sched.add_request(b)
    first = sched.schedule()
    assert [p.request for p in first.portions] == [a, b]
    with pytest.raises(ValueError):
        Scheduler(roomy, 64, 256, admission_headroom=-1)


def test_request_too_large_for_the_pool_fails_alone():
    runner = FakeRunner(num_pages=4, page=4, slots=4)  # 3 usable pages = 12 tokens
    sched = Scheduler(runner, 64, 256)
    small, big, small2 = req(4, new=3), req(20, new=2), req(3, new=2)
    for r in (small, big, small2):
        sched.add_request(r)
    drive(sched, runner)
    assert big.error is not None and "too small" in str(big.error) and big.state is RequestState.FINISHED
    assert small.error is None and small2.error is None
    assert len(small.output_tokens) == 3 and len(small2.output_tokens) == 2
    assert runner.cache.pools[0].num_free == 3


def test_decode_outgrowing_the_pool_alone_fails_with_error():
    runner = FakeRunner(num_pages=3, page=4, slots=2)  # 8 tokens
    sched = Scheduler(runner, 64, 256)
    r = req(6, new=10)
    sched.add_request(r)
    drive(sched, runner)
    assert r.error is not None and len(r.output_tokens) == 3  # positions 6, 7 fit; the 9th token has no page
    assert runner.cache.pools[0].num_free == 2


def test_fail_all_gives_everything_back():
    runner = FakeRunner()
    sched = Scheduler(runner, 8, 256)
    reqs = [req(20), req(5), req(7)]
    for r in reqs:
        sched.add_request(r)
    plan = sched.schedule(); sched.update(plan, runner.run(plan))
    failed = sched.fail_all(RuntimeError("boom"))
    assert len(failed) == 3 and all(isinstance(r.error, RuntimeError) for r in reqs)
    assert not sched.has_work() and runner.cache.live_requests() == []
    runner.cache.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_and_return_all_pages(seed):
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    runner = FakeRunner(num_pages=rng.choice([12, 20, 40]), page=page, slots=rng.choice([2, 4]),
                        window=rng.choice([None, 9]))
    sched = Scheduler(runner, rng.choice([5, 16, 64]), 256)
    reqs = [req(rng.randint(1, 30), new=rng.randint(1, 12)) for _ in range(14)]
    pending = list(reqs)
    steps = 0
    while pending or sched.has_work():
        if pending and rng.random() < 0.4:
            sched.add_request(pending.pop(0))
        if sched.has_work():
            plan = sched.schedule()
            assert plan.num_tokens <= sched.max_num_batched_tokens
            sched.update(plan, runner.run(plan))
            runner.cache.check()
        steps += 1
        assert steps < 5000
    for r in reqs:
        assert r.state is RequestState.FINISHED
        if r.error is None:
            n = len(r.prompt_tokens)
            assert r.output_tokens == [1000 + n + i for i in range(r.params.max_new_tokens)]
    assert runner.cache.live_requests() == []
    assert runner.cache.pools[0].num_free == runner.cache.pools[0].num_pages - 1
    assert 0 < sched.stats.peak_pages <= runner.cache.pools[0].num_pages - 1  # the pool's high-water mark


def test_state_only_model_schedules_by_slots_alone():
    """A model whose every mixer keeps fixed-size state has no page pool: admission is bounded
    by slots, prompts are still cut by the budget, a preempted request is recomputed from its
    first token (its state row is cleared when it is admitted again)."""
    runner = FakeRunner(slots=2)
    runner.cache = CacheManager([], 4, 2, 256)
    sched = Scheduler(runner, max_num_batched_tokens=8, max_seq_len=256)
    reqs = [req(13, new=3), req(5, new=2), req(9, new=4)]
    for r in reqs:
        sched.add_request(r)
    plan = sched.schedule()
    assert [(p.request is reqs[0], p.length) for p in plan.portions] == [(True, 8)]
    sched.update(plan, runner.run(plan))
    plan = sched.schedule()  # the rest of the first prompt, then the second request in the same step
    assert [(reqs.index(p.request), p.start, p.length) for p in plan.portions] == [(0, 8, 5), (1, 0, 3)]
    sched.update(plan, runner.run(plan))
    assert reqs[2].state is RequestState.WAITING  # no slot left
    sched._preempt(reqs[1])  # what a scheduler does when it must take a request's place away
    assert reqs[1].num_computed == 0 and sched.waiting[0] is reqs[1]
    drive(sched, runner)
    for r in reqs:
        n = len(r.prompt_tokens)
        assert r.error is None and r.output_tokens == [1000 + n + i for i in range(r.params.max_new_tokens)]
    assert runner.cache.live_requests() == [] and runner.cache.num_free_slots == 2
