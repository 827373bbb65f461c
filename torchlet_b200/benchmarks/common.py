"""What the benchmarks share: the layer sizes of Qwen2.5-7B (the benchmark model), 14B and 0.5B,
a model of them with random bfloat16 weights made on the GPU, and a cache filled with random keys
and values."""
from __future__ import annotations

import torch

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 152064, "hidden_size": 3584, "intermediate_size": 18944,
    "num_hidden_layers": 28, "num_attention_heads": 28, "num_key_value_heads": 4, "max_position_embeddings": 32768,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": False,
}


QWEN25_14B = {
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 152064, "hidden_size": 5120, "intermediate_size": 13824,
    "num_hidden_layers": 48, "num_attention_heads": 40, "num_key_value_heads": 8, "max_position_embeddings": 32768,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": False,
}
QWEN25_05B = {
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 151936, "hidden_size": 896, "intermediate_size": 4864,
    "num_hidden_layers": 24, "num_attention_heads": 14, "num_key_value_heads": 2, "max_position_embeddings": 32768,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": True,
}
SIZES = {"7b": (QWEN25_7B, 4), "14b": (QWEN25_14B, 6), "0.5b": (QWEN25_05B, 5)}  # layer sizes and the seed of their weights


def build_model(cfg: dict, layers: int, seed: int):
    """The model of ``cfg`` with ``layers`` layers and seeded random bfloat16 weights on cuda:0."""
    from ..config import Qwen2Config
    from ..engine.loading import build_model as build
    from ..weights import random_tensors

    config = Qwen2Config.from_dict(dict(cfg, num_hidden_layers=layers))
    tensors = random_tensors(config, seed, std=0.02, norm_std=0.0, dtype="bfloat16", device="cuda:0")
    model = build(config, tensors, "bfloat16")
    del tensors
    torch.cuda.empty_cache()
    return model


def fill_context(runner, ids, context: int, seed: int) -> None:
    """Admit the requests ``ids`` and give each ``context`` cached tokens of seeded random keys
    and values (the pages are filled in chunks, so that no large temporary is needed)."""
    generator = torch.Generator(device="cuda:0").manual_seed(seed)
    for pages in runner.storage.pages:
        flat = pages.view(-1)
        step = 1 << 27
        for start in range(0, flat.numel(), step):
            chunk = flat[start:start + step]
            chunk.copy_(torch.randn(chunk.shape, generator=generator, device=pages.device, dtype=torch.float32).mul_(0.5))
    for rid in ids:
        runner.admit(rid)
        if not runner.cache.extend(rid, context):
            raise RuntimeError("the page pool is too small for the benchmark's context")
        runner.cache.advance(rid, context)
