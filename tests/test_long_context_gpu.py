"""A request of 6,000 tokens against the plain implementation, position by position: prompt
portions of thousands of tokens behind thousands of cached ones (several waves of the prompt
attention's CTAs, hundreds of pages in a block table), then decoding with the keys split over
dozens of CTAs, beside a short request; in bfloat16 (tensor-core kernels) and in float32."""
import pytest
import torch

import harness
from harness import assert_close, make_runner, plain_logits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_six_thousand_tokens(dtype):
    from torchlet_b200.engine import StepEntry

    length, tail = 6000, 40
    ids, want = plain_logits("G", length, 77)
    other, want_other = plain_logits("G", 300, 78)
    runner = make_runner("G", dtype, num_pages=420, slots=2, budget=4096, max_seq_len=8192)
    runner.admit("long"); runner.admit("short")
    got, got_other = [], []
    fed = fed_other = 0
    with harness.KernelCalls() as calls:
        # the long prompt in three portions, the short request's prompt beside the second
        for size, size_other in ((3000, 0), (2500, 260), (length - tail - 5500, 0)):
            entries = [StepEntry("long", ids[fed:fed + size], list(range(size)))]
            if size_other:
                entries.append(StepEntry("short", other[:size_other], list(range(size_other))))
            logits = runner.step(entries).cpu()
            got.append(logits[:size].clone())
            if size_other:
                got_other.append(logits[size:].clone())
            fed, fed_other = fed + size, fed_other + size_other
        for _ in range(tail):  # both decode, one token each
            logits = runner.step([StepEntry("long", ids[fed:fed + 1], [0]),
                                  StepEntry("short", other[fed_other:fed_other + 1], [0])]).cpu()
            got.append(logits[:1].clone()); got_other.append(logits[1:].clone())
            fed, fed_other = fed + 1, fed_other + 1
    assert fed == length and fed_other == 300
    assert_close(torch.cat(got), want, dtype, "6,000 tokens")
    assert_close(torch.cat(got_other), want_other, dtype, "the short request beside them")
    if dtype == "bfloat16":
        assert calls.counts["attention_generic"] == 0 and calls.counts["attention_tc"] > 0
        assert max(calls.decode_splits) >= 32, calls.decode_splits  # the keys of a decode step over dozens of CTAs
    runner.finish("long"); runner.finish("short")
    runner.cache.check()
    assert runner.cache.live_requests() == []
