"""Configurations at the edges of what config.json allows: head sizes in steps of 16 up to 256,
one to thirty-two query heads a KV head, a width and a vocabulary that are no power of two (nor
multiples of 8), a projection width that differs from the model width (``head_dim`` key), windows
of one token and of less than a page, tied and untied heads, with and without QKV bias.  Every one
through the engine in both dtypes, in portions and token by token, against the plain implementation.
Sizes a tensor-core kernel does not take must fall to the any-size kernels, never to a wrong result."""
import pytest
import torch

import plain_model
import tiny_configs
from harness import assert_close

pytestmark = pytest.mark.gpu


def _config(**over):
    base = {"architectures": ["Qwen2ForCausalLM"], "vocab_size": 300, "hidden_size": 128, "intermediate_size": 96,
            "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 512,
            "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": False}
    base.update(over)
    return base


ODD = {
    "width_100_head_16": _config(hidden_size=100, head_dim=16, num_attention_heads=5, num_key_value_heads=5,
                                 intermediate_size=70, vocab_size=257),
    "head_80_group_2": _config(hidden_size=160, num_attention_heads=2, num_key_value_heads=1, vocab_size=1000,
                               intermediate_size=300, rms_norm_eps=1e-5),
    "head_112_no_bias_tied": _config(hidden_size=336, num_attention_heads=3, num_key_value_heads=3, vocab_size=259,
                                     intermediate_size=72, attention_bias=False, tie_word_embeddings=True),
    "head_256": _config(hidden_size=512, num_attention_heads=2, num_key_value_heads=1, intermediate_size=136,
                        rope_theta=1000000.0),
    "head_128_group_16": _config(hidden_size=256, head_dim=128, num_attention_heads=16, num_key_value_heads=1,
                                 intermediate_size=264, vocab_size=515),
    "head_64_group_32": _config(hidden_size=192, head_dim=64, num_attention_heads=32, num_key_value_heads=1,
                                intermediate_size=200),
    "head_64_group_1_window_1": _config(hidden_size=512, num_attention_heads=8, num_key_value_heads=8,
                                        use_sliding_window=True, sliding_window=1, max_window_layers=1),
    "head_128_window_5_page_32": _config(hidden_size=384, num_attention_heads=3, num_key_value_heads=1,
                                         use_sliding_window=True, sliding_window=5, max_window_layers=0),
    "head_48_window_37": _config(hidden_size=96, num_attention_heads=2, num_key_value_heads=2, intermediate_size=50,
                                 use_sliding_window=True, sliding_window=37, max_window_layers=1, num_hidden_layers=3),
}
PAGES = {"head_128_window_5_page_32": 32, "head_48_window_37": 8, "head_256": 64, "head_64_group_32": 128}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_configuration(name, dtype):
    from torchlet_b200.config import EngineConfig, Qwen2Config
    from torchlet_b200.engine import ModelRunner, StepEntry
    from torchlet_b200.engine.loading import build_model

    cfg = ODD[name]
    weights = tiny_configs.make_weights(cfg, seed=21, std=0.05, norm_std=0.02, dtype=torch.bfloat16)
    model = build_model(Qwen2Config.from_dict(cfg), weights, dtype)
    page = PAGES.get(name, 16)
    runner = ModelRunner(model, EngineConfig(dtype=dtype, max_decode_slots=3, kv_block_size=page, max_seq_len=384,
                                             max_num_blocks=3 * (384 // page) + 1, cuda_graph=True))
    plain_weights = {k: v.float() for k, v in weights.items()}
    seqs = [tiny_configs.make_ids(cfg, n, seed=70 + i) for i, n in enumerate((190, 131))]
    want = [plain_model.forward_logits(cfg, plain_weights, ids) for ids in seqs]
    got = {0: [], 1: []}
    fed = [0, 0]
    runner.admit("r0"); runner.admit("r1")
    # portions of changing size beside each other, then a stretch token by token (the captured decode step)
    plan = [(77, 2), (2, 60), (1, 1), (40, 1), (1, 30), (3, 1)] + [(1, 1)] * 30
    for sizes in plan:
        entries = []
        for r, size in enumerate(sizes):
            size = min(size, len(seqs[r]) - fed[r])
            if size > 0:
                entries.append((r, StepEntry(f"r{r}", seqs[r][fed[r]:fed[r] + size], list(range(size)))))
        logits = runner.step([e for _, e in entries]).cpu()
        row = 0
        for r, e in entries:
            got[r].append(logits[row:row + len(e.tokens)].clone())
            row += len(e.tokens)
            fed[r] += len(e.tokens)
    assert runner.graph_steps >= 20  # the single-token steps replayed the captured decode step
    for r in range(2):
        assert_close(torch.cat(got[r]), want[r][:fed[r]], dtype, f"{name} request {r}")
    runner.finish("r0"); runner.finish("r1")
    runner.cache.check()
