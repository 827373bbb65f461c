"""The engine against the plain implementation, in 32-bit and in bfloat16, for every
way of cutting the work: each request alone and whole; most of it in one step and the
last 32 tokens one by one; portions of changing size down to two tokens; mixed, up to
four live requests with so few pages that they are used again; long decoding; the first
tokens of a sequence."""
import pytest
import torch

import harness
from harness import assert_close, changing_cuts, make_runner, plain_logits, replay

pytestmark = pytest.mark.gpu

CASES = [(name, dtype) for name in ("A", "B") for dtype in ("float32", "bfloat16")]
LENGTHS = {"A": (5, 17, 33, 90), "B": (1, 9, 24, 40, 131)}


@pytest.mark.parametrize("name, dtype", CASES)
def test_whole_requests_alone(name, dtype):
    runner = make_runner(name, dtype)
    for i, length in enumerate(LENGTHS[name]):
        ids, want = plain_logits(name, length, 100 + i)
        got = replay(runner, f"r{i}", ids, [length])
        assert_close(got, want, dtype, f"{name} whole {length}")


@pytest.mark.parametrize("name, dtype", CASES)
def test_last_32_tokens_one_by_one(name, dtype):
    runner = make_runner(name, dtype)
    length = LENGTHS[name][-1]
    ids, want = plain_logits(name, length, 7)
    got = replay(runner, "r", ids, [length - 32] + [1] * 32)
    assert_close(got, want, dtype, f"{name} decode tail")
    whole = replay(runner, "w", ids, [length])
    if dtype == "float32":  # the 32-bit kernels are cut-invariant to the bit
        assert torch.equal(got, whole)


@pytest.mark.parametrize("name, dtype", CASES)
def test_portions_of_changing_size(name, dtype):
    runner = make_runner(name, dtype)
    length = 150
    ids, want = plain_logits(name, length, 8)
    for seed in (0, 5):
        cuts = changing_cuts(length, seed)
        assert min(cuts) <= 2
        got = replay(runner, f"c{seed}", ids, cuts)
        assert_close(got, want, dtype, f"{name} cuts {cuts[:6]}")


@pytest.mark.parametrize("name, dtype", CASES)
def test_mixed_batches_with_pages_used_again(name, dtype):
    """Up to four live requests: portions of some beside decoded tokens of others, in a
    pool so small that later requests get the pages earlier ones gave back."""
    from torchlet_b200.engine import StepEntry

    page = harness.tiny_configs.ALL[name][1]["page_size"]
    lengths = [70, 45, 96, 33, 61, 80, 52]
    plain = [plain_logits(name, n, 200 + i) for i, n in enumerate(lengths)]
    # pool: enough for about 2.5 of the longest requests, so pages change hands
    num_pages = 1 + sum(-(-n // page) for n in sorted(lengths)[-2:]) + 3 * -(-40 // page)
    runner = make_runner(name, dtype, num_pages=num_pages, slots=4)
    progress = {}  # index -> tokens fed
    collected = {i: [] for i in range(len(lengths))}
    waiting = list(range(len(lengths)))
    step = 0
    pages_seen = {}
    while waiting or progress:
        # admit while a slot is free and the pool could hold the request
        while waiting and len(progress) < 4:
            i = waiting[0]
            need = -(-lengths[i] // page)
            in_use = sum(-(-lengths[j] // page) for j in progress)
            if in_use + need > num_pages - 1:
                break
            waiting.pop(0)
            runner.admit(f"m{i}")
            progress[i] = 0
        entries, meta = [], []
        for order, i in enumerate(sorted(progress)):
            ids = plain[i][0]
            done = progress[i]
            left = lengths[i] - done
            # the first live request decodes one token at a time once past half; the
            # others take portions of changing size
            size = 1 if (done > lengths[i] // 2) else [11, 2, 19, 5, 3][(step + order) % 5]
            size = min(size, left)
            entries.append(StepEntry(f"m{i}", ids[done:done + size], list(range(size))))
            meta.append((i, size))
        assert any(s == 1 for _, s in meta) or step < 12
        logits = runner.step(entries).cpu()
        row = 0
        for i, size in meta:
            collected[i].append(logits[row:row + size].clone())
            row += size
            progress[i] += size
            for p in runner.cache.table(f"m{i}", 0):
                pages_seen.setdefault(p, set()).add(i)
            if progress[i] == lengths[i]:
                runner.finish(f"m{i}")
                del progress[i]
        runner.cache.check()
        step += 1
    assert any(len(users) > 1 for p, users in pages_seen.items() if p), "no page was used again"
    for i, n in enumerate(lengths):
        assert_close(torch.cat(collected[i]), plain[i][1], dtype, f"{name} mixed request {i}")


@pytest.mark.parametrize("name, dtype", CASES)
def test_long_decoding(name, dtype):
    runner = make_runner(name, dtype)
    length = 400
    ids, want = plain_logits(name, length, 9)
    got = replay(runner, "long", ids, [3] + [1] * (length - 3))
    assert_close(got, want, dtype, f"{name} long decode")


@pytest.mark.parametrize("name, dtype", CASES)
def test_first_tokens_of_a_sequence(name, dtype):
    runner = make_runner(name, dtype)
    ids, want = plain_logits(name, 6, 10)
    for cuts in ([1, 1, 1, 1, 1, 1], [1, 2, 3], [2, 1, 1, 2], [6]):
        got = replay(runner, "f", ids, cuts)
        assert_close(got, want, dtype, f"{name} first tokens {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_runs_a_layer_twice_and_shares_a_cache(dtype):
    schedule = ((0, None), (1, None), (0, None), (1, 1))
    runner = make_runner("A", dtype, schedule=schedule)
    ids, want = plain_logits("A", 60, 12, schedule=schedule)
    got = replay(runner, "s", ids, [20, 2, 17, 1, 1, 19])
    assert_close(got, want, dtype, "schedule with repeats")
    assert len(runner.storage.pages[0]) == 3  # three executions own cache layers, one reads another's


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_dim_128_through_the_tensor_core_attention(dtype):
    """Tiny D (head_dim 128, 3 heads a KV head): in bfloat16 prompt portions run on the
    tcgen05 attention kernel and decode on the mma.sync kernel; cut into portions with
    cached context before them, beside a second request."""
    from torchlet_b200.engine import StepEntry

    runner = make_runner("D", dtype, num_pages=80)
    ids, want = plain_logits("D", 420, 21)
    got = replay(runner, "h", ids, [150, 2, 129, 1, 1, 100, 37])
    assert_close(got, want, dtype, "head_dim 128, portions")
    other, want_other = plain_logits("D", 140, 22)
    runner.admit("x"); runner.admit("y")
    a = runner.step([StepEntry("x", ids[:300], [299]), StepEntry("y", other[:1], [0])]).cpu().clone()
    b = runner.step([StepEntry("x", ids[300:301], [0]), StepEntry("y", other[1:140], list(range(139)))]).cpu().clone()
    assert_close(torch.cat([a[:1], b[:1]]), want[[299, 300]], dtype, "request x")
    assert_close(torch.cat([a[1:], b[1:]]), want_other, dtype, "request y")
    runner.finish("x"); runner.finish("y")
    runner.cache.check()
