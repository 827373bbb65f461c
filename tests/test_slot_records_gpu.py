"""The slot records on the device (csrc/slots.cu): a captured decode step reads its lanes'
tokens, positions, sampling words and block-table rows from them and advances them itself, so
the host sends only a small command block a step.  Compared with the plain implementation while
requests join the decode set, leave it for a step that is not replayed from the graph, finish and
hand their slot to another request."""
import pytest
import torch

import harness
from harness import assert_close, make_runner, plain_logits

pytestmark = pytest.mark.gpu


def _records(runner):
    records = runner._records.cpu()
    return {"token": records[0], "position": records[1], "counter": records[2]}


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("B", "bfloat16"), ("D", "bfloat16")])
def test_records_follow_requests_through_joins_eager_steps_and_slot_reuse(name, dtype):
    from torchlet_b200.engine import StepEntry
    from torchlet_b200.sampling import SampleSpec

    runner = make_runner(name, dtype, slots=3, cuda_graph=True, num_pages=120)
    lengths = [120, 61, 75, 48]
    plain = [plain_logits(name, n, 400 + i) for i, n in enumerate(lengths)]
    fed = [0] * 4
    got = [[] for _ in lengths]

    def prompt(i, count):
        ids = plain[i][0]
        logits = runner.step([StepEntry(f"s{i}", ids[fed[i]:fed[i] + count], list(range(count)))]).cpu()
        got[i].append(logits.clone())
        fed[i] += count

    def decode(which, counters):
        entries = [StepEntry(f"s{i}", [plain[i][0][fed[i]]], sample=SampleSpec(0.0, 7 + i, counters[i])) for i in which]
        result = runner.run(entries)
        logits = result.logits.cpu()
        for lane, i in enumerate(which):
            got[i].append(logits[lane:lane + 1].clone())
            fed[i] += 1
            counters[i] += 1
        return result

    counters = [0, 0, 0, 0]
    for i in range(3):
        runner.admit(f"s{i}")
    prompt(0, 40); prompt(1, 30); prompt(2, 20)
    graph_before = runner.graph_steps
    for _ in range(5):
        result = decode([0, 1, 2], counters)
    first_steps = runner.h2d_bytes_last_step
    # the device's records say what the host knows: positions, counters, the tokens it sampled
    rec = _records(runner)
    for lane, i in enumerate([0, 1, 2]):
        slot = runner.cache.slot_of(f"s{i}")
        assert int(rec["position"][slot]) == fed[i] == runner.cache.num_tokens(f"s{i}")
        assert int(rec["counter"][slot]) == counters[i]
        assert int(rec["token"][slot]) == int(result.tokens[lane])
    # request 1 leaves the decode set for a step that is not replayed (a portion of 7 tokens), then returns
    prompt(1, 7)
    for _ in range(3):
        decode([0, 1, 2], counters)
    # request 2 ends; request 3 gets its slot, reads its prompt beside the others' decode steps, then decodes
    while fed[2] < lengths[2]:
        decode([2, 0], counters)  # another order of lanes, another bucket
    slot_of_2 = runner.cache.slot_of("s2")
    runner.finish("s2")
    runner.admit("s3")
    assert runner.cache.slot_of("s3") == slot_of_2
    prompt(3, 25)
    while any(fed[i] < lengths[i] for i in (0, 1, 3)):
        live = [i for i in (3, 0, 1) if fed[i] < lengths[i]]
        decode(live, counters)
    assert runner.graph_steps - graph_before >= 40
    for i, n in enumerate(lengths):
        assert_close(torch.cat(got[i]), plain[i][1], dtype, f"{name} request {i}")
    # a steady decode step sends the command block alone: a few words a lane, whatever the tables' width
    from torchlet_b200 import ops

    groups = max(1, runner.num_groups)
    assert first_steps == 4 * ops.slot_command_words(4, 4 * groups)  # three lanes: the bucket of four
    assert runner.h2d_bytes_last_step == 4 * ops.slot_command_words(1, groups)  # one lane at the end
    assert first_steps < 3 * groups * runner.cache.max_pages_per_request * 4  # less than the lanes' table rows alone
    for i in (0, 1, 3):
        runner.finish(f"s{i}")
    runner.cache.check()


def test_sampled_tokens_are_taken_on_the_device_when_the_host_has_not_seen_them():
    """``feed_previous``: the next step's tokens are the ones the step before sampled, read from
    the slot records; greedy decoding this way equals decoding with the host in between."""
    from torchlet_b200.engine import StepEntry
    from torchlet_b200.sampling import SampleSpec

    outs = []
    for ahead in (False, True):
        runner = make_runner("A", "float32", slots=2, cuda_graph=True)
        prompts = [harness.tiny_configs.make_ids(harness.tiny_configs.TINY_A, n, 500 + i) for i, n in enumerate((12, 29))]
        for i, p in enumerate(prompts):
            runner.admit(f"f{i}")
        first = runner.run([StepEntry(f"f{i}", p, sample=SampleSpec(0.0, 1, 0)) for i, p in enumerate(prompts)])
        tokens = [first.tokens.tolist()]
        for k in range(1, 10):
            last = tokens[-1] if not ahead or k == 1 else [0, 0]  # ahead: the host's tokens are placeholders
            entries = [StepEntry(f"f{i}", [last[i]], sample=SampleSpec(0.0, 1, k)) for i in range(2)]
            result = runner.run(entries, feed_previous=ahead and k > 1)
            tokens.append(result.tokens.tolist())
        outs.append(tokens)
    assert outs[0] == outs[1]
