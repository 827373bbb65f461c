"""Seeded random schedules through the step function against the plain implementation: random
request lengths, admission order, portion sizes (single tokens, two tokens, sizes around a page's
and a window's edge, long portions), random subsets of the live requests in a step, and a pool so
small that pages change hands.  Configurations with a window (pages a window has passed are given
back while the request runs) and with the head sizes of the tensor-core kernels, in both dtypes."""
import random

import pytest
import torch

import harness
from harness import assert_close, make_runner, plain_logits

pytestmark = pytest.mark.gpu

CASES = [("B", "float32"), ("B", "bfloat16"), ("D", "bfloat16"), ("E", "bfloat16"), ("F", "float32"), ("F", "bfloat16")]


def _portion(rng, left, page, window):
    """A portion size that likes edges: one or two tokens, a page or a window give or take one,
    what is left, or anything."""
    choices = [1, 1, 2, page - 1, page, page + 1, 3 * page + 1, left, rng.randint(1, max(1, left))]
    if window:
        choices += [window - 1, window, window + 1]
    return max(1, min(left, rng.choice(choices)))


@pytest.mark.parametrize("seed", [0, 1, 2])
@pytest.mark.parametrize("name, dtype", CASES)
def test_random_schedule(name, dtype, seed):
    from torchlet_b200.engine import StepEntry

    cfg, init = harness.tiny_configs.ALL[name]
    page, window = init["page_size"], cfg.get("sliding_window") if cfg.get("use_sliding_window") else None
    rng = random.Random(1000 * seed + len(name) + ord(name))
    longest = min(cfg["max_position_embeddings"], 620)
    lengths = [rng.choice([rng.randint(1, 40), rng.randint(41, 250), rng.randint(251, longest)]) for _ in range(7)]
    lengths[rng.randrange(7)] = longest  # always one that runs far past a window
    plain = [plain_logits(name, n, 7000 + 10 * seed + i) for i, n in enumerate(lengths)]
    pages_of = lambda n: -(-n // page)
    # room for the two longest requests and a little more: later requests get pages earlier ones gave back
    num_pages = 1 + sum(sorted(pages_of(n) for n in lengths)[-2:]) + 4
    runner = make_runner(name, dtype, num_pages=num_pages, slots=4)
    waiting, live, done = list(range(len(lengths))), {}, {}
    collected = {i: [] for i in range(len(lengths))}
    pages_seen, steps, mixed = {}, 0, 0
    with harness.KernelCalls() as calls:
        while waiting or live:
            while waiting and len(live) < 4:
                i = waiting[0]
                if sum(pages_of(lengths[j]) for j in live) + pages_of(lengths[i]) > num_pages - 1:
                    break
                waiting.pop(0)
                runner.admit(f"q{i}")
                live[i] = 0
            # a random, non-empty subset of the live requests runs in this step
            chosen = [i for i in sorted(live) if rng.random() < 0.7] or [rng.choice(sorted(live))]
            rng.shuffle(chosen)
            entries, meta = [], []
            for i in chosen:
                ids, fed = plain[i][0], live[i]
                decoding = fed > 0 and rng.random() < 0.5
                size = 1 if decoding else _portion(rng, lengths[i] - fed, page, window)
                entries.append(StepEntry(f"q{i}", ids[fed:fed + size], list(range(size))))
                meta.append((i, size))
            mixed += any(s == 1 for _, s in meta) and any(s > 1 for _, s in meta)
            logits = runner.step(entries).cpu()
            row = 0
            for i, size in meta:
                collected[i].append(logits[row:row + size].clone())
                row += size
                live[i] += size
                for p in runner.cache.table(f"q{i}", 0):
                    pages_seen.setdefault(int(p), set()).add(i)
                if live[i] == lengths[i]:
                    runner.finish(f"q{i}")
                    del live[i]
            runner.cache.check()
            steps += 1
            assert steps < 5000
    assert mixed > 0 and any(len(users) > 1 for p, users in pages_seen.items() if p), "the schedule was too tame"
    for i, n in enumerate(lengths):
        assert_close(torch.cat(collected[i]), plain[i][1], dtype, f"{name} seed {seed} request {i} ({n} tokens)")
    assert runner.cache.live_requests() == []
    if dtype == "bfloat16" and name in "DEF":
        c = calls.counts
        assert c["attention_generic"] == 0 and c["attention_tc"] > 0 and c["attention_mma"] > 0, c
