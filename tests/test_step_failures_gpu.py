"""A kernel wrapper that raises in the middle of a step of the REAL step function (a prompt
portion, a mixed step, a captured decode step's capture): the engine fails its live requests,
gives everything back, and then generates for new requests exactly what a fresh engine
generates: nothing of the broken step (an unfinished sum left for a later kernel, the device's
slot records, a half-built batch) leaks into the next one."""
import pytest
import torch

import harness
import tiny_configs

pytestmark = pytest.mark.gpu


class Boom(RuntimeError):
    pass


def _engine(name, dtype, graph):
    from torchlet_b200.config import EngineConfig, Qwen2Config
    from torchlet_b200.engine.engine import Engine
    from torchlet_b200.engine.loading import build_model

    cfg, w = harness.weights_for(name)
    model = build_model(Qwen2Config.from_dict(cfg), {k: v.to(torch.bfloat16) for k, v in w.items()}, dtype)
    page = tiny_configs.ALL[name][1]["page_size"]
    return Engine(model, EngineConfig(dtype=dtype, max_decode_slots=4, kv_block_size=page, max_seq_len=256,
                                      max_num_batched_tokens=48, cuda_graph=graph))


def _requests(name, seed):
    from torchlet_b200.engine.scheduler import Request
    from torchlet_b200.sampling import SamplingParams

    cfg = tiny_configs.ALL[name][0]
    return [Request(tiny_configs.make_ids(cfg, n, seed=seed + i), SamplingParams(max_new_tokens=6 + i, ignore_eos=True))
            for i, n in enumerate((70, 9, 33))]


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("name, dtype, op, nth", [
    ("E", "bfloat16", "gemm_tc_deferred", 3), ("E", "bfloat16", "gemm_tc_deferred", 11), ("E", "bfloat16", "gemm_tc", 2),
    ("E", "bfloat16", "finish_accum_norm", 5), ("E", "bfloat16", "attention_tc", 2), ("E", "bfloat16", "attention_mma", 3),
    ("E", "bfloat16", "finish_qkv_rope", 2), ("A", "float32", "gemm_simt", 7), ("A", "float32", "attention_generic", 4),
])
def test_a_step_that_breaks_in_the_middle_leaves_nothing_behind(name, dtype, op, nth, graph):
    from torchlet_b200 import ops
    from torchlet_b200.engine.scheduler import RequestState

    want = [list(r.output_tokens) for r in _engine(name, dtype, graph).generate(_requests(name, 900))]
    engine = _engine(name, dtype, graph)
    original, calls = getattr(ops, op), [0]

    def breaking(*args, **kwargs):
        calls[0] += 1
        if calls[0] == nth:
            raise Boom(f"{op} call {nth}")
        return original(*args, **kwargs)

    setattr(ops, op, breaking)
    try:
        doomed = _requests(name, 400)
        with pytest.raises(Boom):
            engine.generate(doomed)
    finally:
        setattr(ops, op, original)
    assert calls[0] >= nth, "the wrapper was never reached: the case tests nothing"
    assert all(r.state is RequestState.FINISHED for r in doomed) and any(isinstance(r.error, Boom) for r in doomed)
    engine.runner.cache.check()
    assert engine.runner.cache.live_requests() == [] and engine.runner.cache.num_free_slots == 4
    assert ops.workspace_holder is None
    again = engine.generate(_requests(name, 900))
    assert [list(r.output_tokens) for r in again] == want
    engine.runner.cache.check()


def test_a_wait_that_gave_up_inside_a_kernel_fails_the_step_not_the_engine():
    """A bounded wait that runs out leaves a code on the device (here left by the self-test kernel,
    whose wait nothing ends: no fault, no hang).  The engine reads the codes before it hands a
    finished request back, fails what is live instead of returning tokens of a kernel that gave
    up, and serves the next requests as if nothing had been."""
    from torchlet_b200 import ops
    from torchlet_b200.engine.scheduler import RequestState

    want = [list(r.output_tokens) for r in _engine("E", "bfloat16", True).generate(_requests("E", 900))]
    engine = _engine("E", "bfloat16", True)
    ops.wait_selftest(77)
    doomed = _requests("E", 400)
    with pytest.raises(ops.KernelError, match="77"):
        engine.generate(doomed)
    assert all(r.state is RequestState.FINISHED for r in doomed) and all(r.error is not None for r in doomed)
    engine.runner.cache.check()
    assert engine.runner.cache.live_requests() == []
    assert [list(r.output_tokens) for r in engine.generate(_requests("E", 900))] == want
