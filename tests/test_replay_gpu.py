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

# A and B: the two tiny configurations (SIMT kernels in both dtypes: head_dim 16 and 32).  D and E
# (head_dim 128 with 3 heads a KV head, head_dim 64 with 7) and F (head_dim 128, a window of 150 on two
# of three layers): in bfloat16 every cut below runs
# through the tensor-core attention kernels, the tcgen05 products and the fused finishing kernels.
CASES = [(name, dtype) for name in ("A", "B") for dtype in ("float32", "bfloat16")] + [
    ("D", "bfloat16"), ("E", "bfloat16"), ("E", "float32"), ("F", "bfloat16"), ("F", "float32")]
TENSOR_CORE = {("D", "bfloat16"), ("E", "bfloat16"), ("F", "bfloat16")}
LENGTHS = {"A": (5, 17, 33, 90), "B": (1, 9, 24, 40, 131), "D": (3, 40, 200), "E": (1, 70, 259), "F": (2, 149, 151, 420)}


def check_kernels(calls, name, dtype, prompt: bool, decode: bool):
    """The comparison went through the kernels it is meant to cover."""
    if (name, dtype) not in TENSOR_CORE:
        return
    c = calls.counts
    assert c["attention_generic"] == 0 and c["gemm_simt"] == 0, c
    assert c["gemm_tc"] + c["gemm_tc_deferred"] > 0, c
    if prompt:  # prompt portions on the tcgen05 attention (head_dim 128 and 64)
        assert c["attention_tc"] > 0 and c["attention_mma"] == len(calls.decode_splits), c
    if decode:
        assert calls.decode_splits, c
        assert c["finish_qkv_rope"] > 0 and c["finish_accum_norm"] > 0, c


@pytest.mark.parametrize("name, dtype", CASES)
def test_whole_requests_alone(name, dtype):
    runner = make_runner(name, dtype)
    with harness.KernelCalls() as calls:
        for i, length in enumerate(LENGTHS[name]):
            ids, want = plain_logits(name, length, 100 + i)
            got = replay(runner, f"r{i}", ids, [length])
            assert_close(got, want, dtype, f"{name} whole {length}")
    check_kernels(calls, name, dtype, prompt=True, decode=False)


@pytest.mark.parametrize("name, dtype", CASES)
def test_last_32_tokens_one_by_one(name, dtype):
    runner = make_runner(name, dtype)
    length = LENGTHS[name][-1]
    ids, want = plain_logits(name, length, 7)
    with harness.KernelCalls() as calls:
        got = replay(runner, "r", ids, [length - 32] + [1] * 32)
    assert_close(got, want, dtype, f"{name} decode tail")
    check_kernels(calls, name, dtype, prompt=True, decode=True)
    if (name, dtype) in TENSOR_CORE:
        assert max(calls.decode_splits) > 1, "the keys of a decode step were never split over CTAs"
    whole = replay(runner, "w", ids, [length])
    if dtype == "float32":  # the 32-bit kernels are cut-invariant to the bit
        assert torch.equal(got, whole)


@pytest.mark.parametrize("name, dtype", CASES)
def test_portions_of_changing_size(name, dtype):
    runner = make_runner(name, dtype)
    length = 150 if (name, dtype) not in TENSOR_CORE else 330
    ids, want = plain_logits(name, length, 8)
    with harness.KernelCalls() as calls:
        for seed in (0, 5):
            cuts = changing_cuts(length, seed)
            assert min(cuts) <= 2
            got = replay(runner, f"c{seed}", ids, cuts)
            assert_close(got, want, dtype, f"{name} cuts {cuts[:6]}")
    check_kernels(calls, name, dtype, prompt=True, decode=True)


@pytest.mark.parametrize("name, dtype", CASES)
def test_mixed_batches_with_pages_used_again(name, dtype):
    """Up to four live requests: portions of some beside decoded tokens of others, in a
    pool so small that later requests get the pages earlier ones gave back."""
    from torchlet_b200.engine import StepEntry

    page = harness.tiny_configs.ALL[name][1]["page_size"]
    lengths = [70, 45, 96, 33, 61, 80, 52]
    if (name, dtype) in TENSOR_CORE:  # long enough that decode steps split their keys over CTAs
        lengths = [4 * n for n in lengths]
    plain = [plain_logits(name, n, 200 + i) for i, n in enumerate(lengths)]
    # pool: enough for about 2.5 of the longest requests, so pages change hands
    num_pages = 1 + sum(-(-n // page) for n in sorted(lengths)[-2:]) + 3 * -(-lengths[3] // page)
    runner = make_runner(name, dtype, num_pages=num_pages, slots=4)
    progress = {}  # index -> tokens fed
    collected = {i: [] for i in range(len(lengths))}
    waiting = list(range(len(lengths)))
    step = mixed_steps = 0
    pages_seen = {}
    with harness.KernelCalls() as calls:
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
                # a live request decodes one token at a time once past half (at most 24 such steps
                # where the requests are long); the others take portions of changing size
                decoding = done > lengths[i] // 2 and (lengths[i] <= 100 or done <= lengths[i] // 2 + 24)
                size = 1 if decoding else [11, 2, 19, 5, 3][(step + order) % 5] * (1 if lengths[i] <= 100 else 3)
                size = min(size, left)
                entries.append(StepEntry(f"m{i}", ids[done:done + size], list(range(size))))
                meta.append((i, size))
            mixed_steps += any(size == 1 for _, size in meta) and any(size > 1 for _, size in meta)
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
    assert mixed_steps >= 10, "portions of prompts hardly ever ran beside decoded tokens"
    for i, n in enumerate(lengths):
        assert_close(torch.cat(collected[i]), plain[i][1], dtype, f"{name} mixed request {i}")
    check_kernels(calls, name, dtype, prompt=True, decode=True)
    if (name, dtype) in TENSOR_CORE:
        assert max(calls.decode_splits) > 1, "the keys of a decode step were never split over CTAs"
        assert calls.side_by_side >= 10, "the decode attention never ran beside the prompt portions' kernel"


@pytest.mark.parametrize("name, dtype", CASES)
def test_long_decoding(name, dtype):
    runner = make_runner(name, dtype)
    length = 400
    ids, want = plain_logits(name, length, 9)
    got = replay(runner, "long", ids, [3] + [1] * (length - 3))
    assert_close(got, want, dtype, f"{name} long decode")


@pytest.mark.parametrize("name, dtype", CASES)
def test_decode_steps_replayed_from_the_cuda_graph(name, dtype):
    """The captured decode graph (static buffers, padded batch, fused finishing kernels, key
    splits planned without the host) against the plain implementation: LOGITS of every decode
    step, not only tokens.  Three requests of different lengths are fed their known tokens."""
    from torchlet_b200.engine import StepEntry
    from torchlet_b200.sampling import SampleSpec

    runner = make_runner(name, dtype, slots=4, cuda_graph=True)
    lengths = (LENGTHS[name][-1], LENGTHS[name][-2] + 20, 30)
    plain = [plain_logits(name, n, 300 + i) for i, n in enumerate(lengths)]
    steps = 24
    for i in range(3):
        runner.admit(f"g{i}")
    runner.step([StepEntry(f"g{i}", plain[i][0][:n - steps], []) for i, n in enumerate(lengths)])
    got = [[] for _ in lengths]
    with harness.KernelCalls() as calls:
        for k in range(steps):
            entries = [StepEntry(f"g{i}", [plain[i][0][n - steps + k]], sample=SampleSpec(0.0, 0, k))
                       for i, n in enumerate(lengths)]
            result = runner.run(entries)
            logits = result.logits.cpu()
            assert result.tokens.tolist() == logits.argmax(-1).tolist()
            for i in range(3):
                got[i].append(logits[i].clone())
    assert runner.graph_steps == steps
    for i, n in enumerate(lengths):
        assert_close(torch.stack(got[i]), plain[i][1][n - steps:], dtype, f"{name} graph decode, request {i}")
    for i in range(3):
        runner.finish(f"g{i}")
    runner.cache.check()


@pytest.mark.parametrize("name, dtype", CASES)
def test_first_tokens_of_a_sequence(name, dtype):
    runner = make_runner(name, dtype)
    ids, want = plain_logits(name, 6, 10)
    for cuts in ([1, 1, 1, 1, 1, 1], [1, 2, 3], [2, 1, 1, 2], [6]):
        got = replay(runner, "f", ids, cuts)
        assert_close(got, want, dtype, f"{name} first tokens {cuts}")


def test_portions_behind_a_long_prefix_share_their_key_tiles():
    """A portion of a prompt behind 1,200 cached tokens has few row tiles for the whole GPU: its
    key tiles are shared by several CTAs and merged (csrc/attention_tc.cu), beside a request that
    decodes.  Tiny D, bfloat16, against the plain implementation."""
    from torchlet_b200.engine import StepEntry

    runner = make_runner("D", "bfloat16", num_pages=160, budget=2048)
    ids, want = plain_logits("D", 1500, 31)
    other, want_other = plain_logits("D", 300, 32)
    runner.admit("long"); runner.admit("short")
    got, got_other = [], []
    with harness.KernelCalls() as calls:
        plan = [(1200, 280), (150, 1), (2, 1), (148, 1)]
        a = b = 0
        for n_long, n_short in plan:
            entries = [StepEntry("long", ids[a:a + n_long], list(range(n_long))),
                       StepEntry("short", other[b:b + n_short], list(range(n_short)))]
            logits = runner.step(entries).cpu()
            got.append(logits[:n_long].clone()); got_other.append(logits[n_long:].clone())
            a += n_long; b += n_short
    assert max(calls.prompt_splits) > 1, "no portion's key tiles were ever shared"
    assert_close(torch.cat(got), want, "bfloat16", "portions behind a long prefix")
    assert_close(torch.cat(got_other), want_other[:b], "bfloat16", "the request beside them")
    runner.finish("long"); runner.finish("short")
    runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_runs_a_layer_twice_and_shares_a_cache(dtype):
    schedule = ((0, None), (1, None), (0, None), (1, 1))
    runner = make_runner("A", dtype, schedule=schedule)
    ids, want = plain_logits("A", 60, 12, schedule=schedule)
    got = replay(runner, "s", ids, [20, 2, 17, 1, 1, 19])
    assert_close(got, want, dtype, "schedule with repeats")
    assert len(runner.storage.pages[0]) == 3  # three executions own cache layers, one reads another's


@pytest.mark.parametrize("page", [8, 32, 64, 128])
@pytest.mark.parametrize("name", ["D", "F"])
def test_other_page_sizes_on_the_tensor_core_kernels(name, page):
    """Pages of 8 to 128 tokens (what the TMA page boxes of both attention kernels take), with and
    without a window: whole, a decode tail replayed from the captured step, and changing portions."""
    length = LENGTHS[name][-1]
    runner = make_runner(name, "bfloat16", num_pages=max(16, 3 * -(-length // page)), page_size=page, cuda_graph=True)
    ids, want = plain_logits(name, length, 7)
    with harness.KernelCalls() as calls:
        for cuts in ([length], [length - 32] + [1] * 32, changing_cuts(length, seed=page)):
            assert_close(replay(runner, "r", ids, cuts), want, "bfloat16", f"{name}, pages of {page}, {len(cuts)} portions")
    assert calls.counts["attention_generic"] == 0 and calls.counts["attention_tc"] > 0 and calls.decode_splits
    assert runner.graph_steps > 0


@pytest.mark.parametrize("graph", [False, True])
def test_schedule_with_a_shared_cache_on_the_tensor_core_kernels(graph):
    """The same schedule at tiny E's sizes in bfloat16: the execution that reads another one's cache
    rotates its q but writes no keys or values (the fused finishing kernel's store is off), in
    eager steps and in steps replayed from the captured decode step."""
    schedule = ((0, None), (1, None), (0, None), (1, 1))
    runner = make_runner("E", "bfloat16", schedule=schedule, cuda_graph=graph)
    ids, want = plain_logits("E", 150, 13, schedule=schedule)
    with harness.KernelCalls() as calls:
        got = replay(runner, "s", ids, [70, 2, 45, 1] + [1] * 32)
    assert_close(got, want, "bfloat16", "schedule with repeats, tensor-core kernels")
    assert calls.counts["attention_generic"] == 0 and calls.counts["finish_qkv_rope"] > 0
    assert (runner.graph_steps > 0) == graph
    assert len(runner.storage.pages[0]) == 3


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
