"""The engine on memory full of NaN: before the step function is built, and again before every
replay, device memory is filled with NaN and handed back to the caching allocator, so that every
``torch.empty`` scratch buffer, workspace and staging area starts as NaN.  Whatever a kernel
reads without having written it (a row past the step's tokens, a workspace plane no split wrote,
the tail of a buffer sized for the token budget) then shows as NaN in the logits.  Eager steps and
steps replayed from the captured decode step, both dtypes."""
import pytest
import torch

import harness
from harness import assert_close, changing_cuts, make_runner, plain_logits, replay

pytestmark = pytest.mark.gpu


def poison(total_mb: int) -> None:
    blocks, left, i = [], total_mb << 20, 0
    sizes = [1 << 12, 1 << 16, 1 << 20, 1 << 22, 1 << 24, 1 << 26]  # the allocator keeps small and large blocks apart
    while left > 0:
        blocks.append(torch.full((sizes[i % len(sizes)] // 4,), float("nan"), device="cuda"))
        left -= sizes[i % len(sizes)]
        i += 1
    del blocks  # back to the caching allocator, still NaN
    for n in (1 << 10, 1 << 18, 1 << 23):  # (a block may be carved from a larger one that was never filled: most, not all)
        share = torch.isnan(torch.empty(n, device="cuda")).float().mean().item()
        assert share > 0.5, "the allocator did not hand the poisoned memory back"


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("name, dtype, length", [("A", "float32", 90), ("B", "bfloat16", 131), ("D", "bfloat16", 200),
                                                 ("E", "bfloat16", 259), ("F", "bfloat16", 420), ("F", "float32", 420)])
def test_scratch_memory_full_of_nan(name, dtype, length, graph):
    poison(2000)
    runner = make_runner(name, dtype, cuda_graph=graph)
    ids, want = plain_logits(name, length, 7)
    for cuts in ([length], [length - 32] + [1] * 32, changing_cuts(length)):
        poison(300)
        got = replay(runner, "r", ids, cuts)
        assert torch.isfinite(got).all(), f"{len(cuts)} portions: NaN from memory nobody wrote reached the logits"
        assert_close(got, want, dtype, f"{name} {len(cuts)} portions on poisoned memory")
    if graph:
        assert runner.graph_steps > 0
