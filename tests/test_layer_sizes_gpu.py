"""The engine at Qwen2.5-7B LAYER SIZES (hidden 3584, 28 heads in 4 groups of 7, head_dim 128,
intermediate 18944, vocabulary 152064, untied LM head), one layer, random weights: logits of a
40-token sequence against the plain implementation for three ways of cutting it into steps,
in float32 and in bfloat16.  These are the sizes the benchmark runs, so the kernels are the
ones it times (tcgen05 products and attention, the fused finishing kernels of single-token
steps)."""
import pytest
import torch

import harness
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 152064, "hidden_size": 3584, "intermediate_size": 18944,
    "num_hidden_layers": 1, "num_attention_heads": 28, "num_key_value_heads": 4, "max_position_embeddings": 256,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": False,
}
LENGTH = 40
CUTS = {"whole": [40], "last tokens one by one": [33] + [1] * 7, "portions": [5, 2, 17, 3, 13]}


@pytest.fixture(scope="module")
def case():
    weights = tiny_configs.make_weights(CONFIG, seed=21, std=0.02, norm_std=0.02, dtype=torch.bfloat16)
    ids = tiny_configs.make_ids(CONFIG, LENGTH, seed=22)
    # in float64 (sums of 18,944 terms), so that the CPU's own float32 rounding is no part of the comparison
    plain = plain_model.forward_logits(CONFIG, {k: v.float() for k, v in weights.items()}, ids, dtype=torch.float64)
    return weights, ids, plain.float()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logits_at_benchmark_layer_sizes(case, dtype):
    from torchlet_b200.config import EngineConfig, Qwen2Config
    from torchlet_b200.engine import ModelRunner
    from torchlet_b200.engine.loading import build_model

    weights, ids, plain = case
    model = build_model(Qwen2Config.from_dict(CONFIG), weights, dtype)
    runner = ModelRunner(model, EngineConfig(dtype=dtype, max_decode_slots=2, kv_block_size=16, max_num_blocks=12,
                                             max_seq_len=64, max_num_batched_tokens=64, cuda_graph=False))
    limit = harness.TOLERANCE[dtype] * plain.abs().max()
    results = {}
    for name, cuts in CUTS.items():
        got = harness.replay(runner, name, ids, cuts)
        assert (got - plain).abs().max() <= limit, f"{dtype}, {name}: {(got - plain).abs().max()} > {limit}"
        results[name] = got
    if dtype == "float32":  # the 32-bit path does not depend on the cut at all
        assert torch.equal(results["whole"], results["portions"])
        assert torch.equal(results["whole"], results["last tokens one by one"])
    runner.cache.check()


def test_a_long_portion_in_bfloat16_against_the_32_bit_path(case):
    """704 tokens in one step: the products run on the CTA-pair kernel (three 256-row tiles),
    the attention over several key tiles with two row tiles a CTA.  The 32-bit path of the
    engine (checked against the plain implementation above and in the other tests) is the
    reference here: the plain implementation would need minutes for this on the CPU."""
    from torchlet_b200.config import EngineConfig, Qwen2Config
    from torchlet_b200.engine import ModelRunner, StepEntry
    from torchlet_b200.engine.loading import build_model

    weights, _, _ = case
    ids = tiny_configs.make_ids(CONFIG, 704, seed=23)
    want_rows = [0, 1, 127, 128, 300, 511, 512, 639, 703]
    got = {}
    for dtype in ("float32", "bfloat16"):
        model = build_model(Qwen2Config.from_dict(dict(CONFIG, max_position_embeddings=1024)), weights, dtype)
        runner = ModelRunner(model, EngineConfig(dtype=dtype, max_decode_slots=2, kv_block_size=16, max_num_blocks=50,
                                                 max_seq_len=768, max_num_batched_tokens=704, cuda_graph=False))
        runner.admit("p")
        got[dtype] = runner.step([StepEntry("p", ids, want_rows)]).cpu().clone()
        # eight more tokens one by one, from the cache the long step left
        tail = []
        for token in tiny_configs.make_ids(CONFIG, 8, seed=24):
            tail.append(runner.step([StepEntry("p", [token], [0])]).cpu().clone())
        got[dtype] = torch.cat([got[dtype]] + tail)
        runner.finish("p")
        runner.cache.check()
        del runner, model
        torch.cuda.empty_cache()
    harness.assert_close(got["bfloat16"], got["float32"], "bfloat16", "704 tokens and 8 decoded")
    from torchlet_b200 import ops

    ops.raise_on_wait_errors()


@pytest.mark.parametrize("batch", [8, 40])
def test_requests_decoding_together_at_benchmark_layer_sizes(case, batch):
    """``batch`` requests decode together for six steps, replayed from the captured step (the
    16- and 64-token tiles of the weight-streaming products, their K splits and the fused
    finishing kernels at the real widths, the decode attention of many requests at once):
    bfloat16 against the engine's 32-bit path, every request's logits of every step."""
    from torchlet_b200.config import EngineConfig, Qwen2Config
    from torchlet_b200.engine import ModelRunner, StepEntry
    from torchlet_b200.engine.loading import build_model

    weights, _, _ = case
    lengths = [3 + (7 * i) % 29 for i in range(batch)]
    prompts = [tiny_configs.make_ids(CONFIG, n + 6, seed=300 + i) for i, n in enumerate(lengths)]
    got = {}
    for dtype in ("float32", "bfloat16"):
        model = build_model(Qwen2Config.from_dict(CONFIG), weights, dtype)
        runner = ModelRunner(model, EngineConfig(dtype=dtype, max_decode_slots=batch, kv_block_size=16, max_seq_len=64,
                                                 max_num_batched_tokens=2048, cuda_graph=True))
        for i in range(batch):
            runner.admit(f"r{i}")
        runner.step([StepEntry(f"r{i}", prompts[i][:lengths[i]], []) for i in range(batch)])
        steps = []
        for k in range(6):
            steps.append(runner.step([StepEntry(f"r{i}", [prompts[i][lengths[i] + k]], [0]) for i in range(batch)]).cpu().clone())
        assert runner.graph_steps == 6
        got[dtype] = torch.cat(steps)
        for i in range(batch):
            runner.finish(f"r{i}")
        runner.cache.check()
        del runner, model
        torch.cuda.empty_cache()
    harness.assert_close(got["bfloat16"], got["float32"], "bfloat16", f"{batch} requests decoding together")
    from torchlet_b200 import ops

    ops.raise_on_wait_errors()
