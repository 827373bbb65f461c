"""What the step function refuses, in words, and that it can be used afterwards: a request twice
in a step, a token id outside the vocabulary (eager and captured decode steps), a wanted place
outside a request's tokens, more tokens than the budget, no pages left; a prompt kernel for the
page sizes the tcgen05 attention does not take."""
import pytest
import torch

import harness
from harness import assert_close, make_runner, plain_logits, replay

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("graph", [False, True])
def test_bad_steps_are_refused_and_the_next_good_step_runs(graph):
    from torchlet_b200.engine import StepEntry
    from torchlet_b200.engine.runner import OutOfPages

    runner = make_runner("A", "float32", num_pages=5, slots=3, budget=64, cuda_graph=graph)
    vocab = harness.tiny_configs.ALL["A"][0]["vocab_size"]
    ids, want = plain_logits("A", 40, 3)
    runner.admit("a"); runner.admit("b")
    first = runner.step([StepEntry("a", ids[:20], [19])]).cpu().clone()
    with pytest.raises(ValueError, match="twice"):
        runner.step([StepEntry("a", ids[20:21], [0]), StepEntry("a", ids[21:22], [0])])
    with pytest.raises(ValueError, match="token ids"):
        runner.step([StepEntry("a", [vocab], [0])])            # a single token: the captured step's check when graph
    with pytest.raises(ValueError, match="token ids"):
        runner.step([StepEntry("a", [3, -1, 5], [2])])         # a portion: the eager step's check
    with pytest.raises(ValueError, match="outside"):
        runner.step([StepEntry("a", ids[20:23], [3])])
    with pytest.raises(ValueError, match="budget"):
        runner.step([StepEntry("b", [1] * 65, [])])
    with pytest.raises(OutOfPages):                             # 4 usable pages of 16 tokens: a has two, b asks for four
        runner.step([StepEntry("b", [1] * 60, []), StepEntry("a", ids[20:21], [0])])
    runner.cache.check()
    assert runner.cache.num_tokens("a") == 20 and runner.cache.num_tokens("b") == 0
    # nothing of the refused steps has reached the cache: the request goes on as if they had not been
    rest = [runner.step([StepEntry("a", ids[k:k + 1], [0])]).cpu().clone() for k in range(20, 40)]
    assert_close(torch.cat([first] + rest), want[19:], "float32", "after refused steps")
    runner.finish("a"); runner.finish("b")
    runner.cache.check()
    if graph:
        assert runner.graph_steps >= 20


def test_page_sizes_the_tcgen05_attention_does_not_take():
    """Pages of 24 tokens do not divide its 128-key tiles: prompt portions run the mma.sync kernel
    of 64-row tiles instead, in every cut; decode keeps its kernel (no TMA boxes: 64 % 24 != 0)."""
    from torchlet_b200 import ops

    assert not ops.attention_tc_supported(128, 3, 24)
    runner = make_runner("D", "bfloat16", num_pages=60, page_size=24)
    ids, want = plain_logits("D", 200, 5)
    with harness.KernelCalls() as calls:
        for cuts in ([200], [168] + [1] * 32, harness.changing_cuts(200)):
            assert_close(replay(runner, "r", ids, cuts), want, "bfloat16", f"page size 24, {len(cuts)} portions")
    assert calls.counts["attention_tc"] == 0 and calls.counts["attention_generic"] == 0
    assert calls.counts["attention_mma"] > len(calls.decode_splits) > 0  # prompt tiles and decode tiles
