"""Continuous batching under load: many requests of random lengths arriving while others
run, greedy and temperature sampling mixed, a page pool too small for all of them.  Every
request must finish, every page and slot must come back, every produced token must be what the
plain implementation gives for the tokens before it (in both dtypes), and in float32 every output
must equal the same request run alone (Qwen2.5-0.5B head geometry: 14 heads in 2 groups of 7,
head_dim 64, so the tensor-core kernels run in the bfloat16 case)."""
import random

import pytest
import torch

import tiny_configs

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 2048, "hidden_size": 896, "intermediate_size": 1216,
    "num_hidden_layers": 2, "num_attention_heads": 14, "num_key_value_heads": 2, "max_position_embeddings": 512,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": True,
}


# the same with a window of 48 tokens on the second layer: two cache groups, pages given back while a request runs
WINDOWED = dict(CONFIG, use_sliding_window=True, sliding_window=48, max_window_layers=1)


def build(dtype, config=CONFIG, **engine):
    from torchlet_b200.config import EngineConfig, Qwen2Config
    from torchlet_b200.engine.engine import Engine
    from torchlet_b200.engine.loading import build_model

    weights = tiny_configs.make_weights(config, seed=5, std=0.02, norm_std=0.01, dtype=torch.bfloat16)
    model = build_model(Qwen2Config.from_dict(config), weights, dtype)
    return Engine(model, EngineConfig(dtype=dtype, max_seq_len=256, **engine))


def check_against_plain(requests, dtype, config=CONFIG):
    """Every produced token against the plain implementation, given the tokens before it: the
    greedy ones must be the plain argmax (within rounding of it in bfloat16), the sampled ones
    the argmax of the plain scores with the request's own noise."""
    import plain_model

    weights = {k: v.float() for k, v in tiny_configs.make_weights(config, seed=5, std=0.02, norm_std=0.01,
                                                                   dtype=torch.bfloat16).items()}
    slack = 0.0 if dtype == "float32" else 2.5e-2
    for request in requests:
        ids = request.prompt_tokens + request.output_tokens
        logits = plain_model.forward_logits(config, weights, ids)
        first = len(request.prompt_tokens) - 1
        temperature = request.params.temperature
        for k, token in enumerate(request.output_tokens):
            row = logits[first + k]
            room = slack * float(row.abs().max()) + 1e-5
            if temperature == 0:
                assert float(row[token]) >= float(row.max()) - room, (request.request_id, k)
            else:
                scores = plain_model.temperature_scores(row, temperature, request.seed, k)
                # (the kernel takes its logarithms in float32, the plain restatement in float64)
                assert scores[token] >= max(scores) - room / temperature - 1e-3, (request.request_id, k)


def make_requests(count, seed):
    from torchlet_b200.engine.scheduler import Request
    from torchlet_b200.sampling import SamplingParams

    rng = random.Random(seed)
    requests = []
    for i in range(count):
        prompt = [rng.randrange(CONFIG["vocab_size"]) for _ in range(rng.randint(4, 150))]
        params = SamplingParams(max_new_tokens=rng.randint(4, 40), temperature=rng.choice([0.0, 0.0, 0.7]), seed=1000 + i)
        requests.append(Request(prompt, params))
    return requests


# The admission rule of the scheduler (pages for all of a request's tokens and a page of headroom
# for every running request) keeps preemptions rare; with it switched off (None) the same pools
# thrash, which is what exercises preemption and recomputation under load.
@pytest.mark.parametrize("headroom", [None, 1])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_requests_arriving_while_others_run(dtype, headroom):
    count = 40
    engine = build(dtype, max_decode_slots=8, kv_block_size=16, max_num_blocks=41, max_num_batched_tokens=96,
                   admission_headroom=headroom)
    requests = make_requests(count, seed=1)
    rng = random.Random(2)
    pending = list(requests)
    steps = 0
    while pending or engine.scheduler.has_work():
        arrivals = min(len(pending), rng.choice([0, 0, 1, 1, 2, 3]))  # a seeded arrival pattern
        if arrivals:
            engine.add_requests([pending.pop(0) for _ in range(arrivals)])
        if engine.scheduler.has_work():
            engine.step()
        engine.runner.cache.check()
        steps += 1
        assert steps < 20000
    stats = engine.scheduler.stats
    assert stats.finished == count and stats.failed == 0
    if headroom is None:
        assert stats.preemptions > 0, "the pool was meant to be too small"
    else:
        assert stats.peak_pages >= 30, "the pool was meant to be nearly full at times"
    assert all(r.error is None and len(r.output_tokens) == r.params.max_new_tokens for r in requests)
    assert engine.runner.cache.live_requests() == []
    assert engine.runner.cache.pools[0].num_free == 40 and engine.runner.cache.num_free_slots == 8
    check_against_plain(requests, dtype)
    if dtype == "float32":
        alone = build(dtype, max_decode_slots=1, kv_block_size=16, max_num_batched_tokens=512)
        again = make_requests(count, seed=1)
        for request, fresh in zip(requests, again):
            alone.generate([fresh])
            assert fresh.output_tokens == request.output_tokens, f"request {request.request_id} depends on its batch"


@pytest.mark.parametrize("headroom", [None, 1])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_with_a_tight_pool_and_stop_tokens(dtype, headroom):
    """``Engine.run`` (one decode step ahead) with everything at once: more requests than
    slots, a pool that forces preemption (also when the step ahead finds no page), stop tokens
    that end requests a step before the host knows.  In float32 every output equals the request
    run alone with synchronous steps."""
    from torchlet_b200.engine.scheduler import Request
    from torchlet_b200.sampling import SamplingParams

    count = 30
    rng = random.Random(11)
    stops = tuple(rng.sample(range(CONFIG["vocab_size"]), 60))  # 3 % of the vocabulary ends a request

    def make():
        r = random.Random(12)
        out = []
        for i in range(count):
            prompt = [r.randrange(CONFIG["vocab_size"]) for _ in range(r.randint(4, 120))]
            out.append(Request(prompt, SamplingParams(max_new_tokens=r.randint(8, 60), temperature=r.choice([0.0, 0.9]),
                                                      seed=500 + i, stop_token_ids=stops)))
        return out

    engine = build(dtype, max_decode_slots=6, kv_block_size=16, max_num_blocks=31, max_num_batched_tokens=128,
                   admission_headroom=headroom)
    requests = make()
    engine.generate(requests)
    engine.runner.cache.check()
    stats = engine.scheduler.stats
    assert stats.finished == count and stats.failed == 0
    if headroom is None:
        assert stats.preemptions > 0, "the pool was meant to be too small"
    else:
        assert stats.peak_pages >= 24, "the pool was meant to be nearly full at times"
    assert engine.steps_ahead > 0
    assert all(r.error is None for r in requests)
    assert any(len(r.output_tokens) < r.params.max_new_tokens for r in requests), "no stop token was drawn"
    assert all(t not in stops for r in requests for t in r.output_tokens)
    assert engine.runner.cache.live_requests() == []
    assert engine.runner.cache.pools[0].num_free == 30 and engine.runner.cache.num_free_slots == 6
    check_against_plain(requests, dtype)
    if dtype == "float32":
        alone = build(dtype, max_decode_slots=1, kv_block_size=16, max_num_batched_tokens=512)
        for request, fresh in zip(requests, make()):
            alone.add_requests([fresh])
            while alone.scheduler.has_work():
                alone.step()
            assert fresh.output_tokens == request.output_tokens, f"request {request.request_id} depends on its batch"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_windowed_layer_under_load(dtype):
    """The loop one step ahead, the captured decode step, a tight pool with preemptions and stop
    tokens, now with a window on one of the two layers: its group gives pages back while requests
    decode, the device's block tables keep the passed entries, and every produced token is still
    the plain implementation's."""
    from torchlet_b200.engine.scheduler import Request
    from torchlet_b200.sampling import SamplingParams

    count = 24
    r = random.Random(21)
    stops = tuple(r.sample(range(WINDOWED["vocab_size"]), 40))
    requests = [Request([r.randrange(WINDOWED["vocab_size"]) for _ in range(r.randint(4, 150))],
                        SamplingParams(max_new_tokens=r.randint(20, 90), temperature=r.choice([0.0, 0.8]), seed=700 + i,
                                       stop_token_ids=stops)) for i in range(count)]
    engine = build(dtype, WINDOWED, max_decode_slots=6, kv_block_size=16, max_num_blocks=36, max_num_batched_tokens=128,
                   admission_headroom=None)
    engine.generate(requests)
    cache = engine.runner.cache
    cache.check()
    stats = engine.scheduler.stats
    assert len(cache.groups) == 2 and {g.window for g in cache.groups} == {None, 48}
    assert stats.finished == count and stats.failed == 0 and stats.preemptions > 0 and engine.steps_ahead > 0
    assert engine.runner.graph_steps > 0 and cache.live_requests() == []
    assert all(pool.num_free == pool.num_pages - 1 for pool in cache.pools)
    assert max(len(q.prompt_tokens) + len(q.output_tokens) for q in requests) > 48 + 64, "nobody ran far past the window"
    check_against_plain(requests, dtype, WINDOWED)
