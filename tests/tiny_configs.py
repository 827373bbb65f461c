"""The two tiny configurations the tests run, differing in every size and option, and
helpers that make their weights.  Plain dicts with config.json's keys."""
from __future__ import annotations

import torch

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 128,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "max_position_embeddings": 512,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": True,
    "tie_word_embeddings": True,
}
TINY_A_INIT = {"seed": 0, "std": 0.02, "norm_std": 0.01, "page_size": 16}

# differs in every size and option: 3 heads in one group (g = 3), head_dim 32, sizes that
# are no power of two, untied head, other theta and eps, and a window on layers 1 and 2
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 384,
    "hidden_size": 96,
    "intermediate_size": 224,
    "num_hidden_layers": 3,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "max_position_embeddings": 640,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5,
    "attention_bias": True,
    "tie_word_embeddings": False,
    "use_sliding_window": True,
    "sliding_window": 40,
    "max_window_layers": 1,
}
TINY_B_INIT = {"seed": 2, "std": 0.03, "norm_std": 0.02, "page_size": 8}

# a third one for kernels and parts at other sizes: head_dim 48 (not a power of two), g = 5
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 331,
    "hidden_size": 240,
    "head_dim": 48,
    "intermediate_size": 200,
    "num_hidden_layers": 2,
    "num_attention_heads": 5,
    "num_key_value_heads": 1,
    "max_position_embeddings": 512,
    "rope_theta": 50000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": False,
    "tie_word_embeddings": False,
}
TINY_C_INIT = {"seed": 5, "std": 0.04, "norm_std": 0.02, "page_size": 32}

# head_dim 128 with 3 query heads a KV head: the shapes the tcgen05 attention kernel takes
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 300,
    "hidden_size": 768,
    "intermediate_size": 320,
    "num_hidden_layers": 2,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "max_position_embeddings": 2048,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": True,
    "tie_word_embeddings": False,
}
TINY_D_INIT = {"seed": 7, "std": 0.02, "norm_std": 0.02, "page_size": 16}

# head_dim 64 with 7 query heads a KV head (the head geometry of the reference's own example
# size), a width and a vocabulary that are no power of two, tied head
TINY_E = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 411,
    "hidden_size": 896,
    "intermediate_size": 304,
    "num_hidden_layers": 2,
    "num_attention_heads": 14,
    "num_key_value_heads": 2,
    "max_position_embeddings": 1024,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": True,
    "tie_word_embeddings": True,
}
TINY_E_INIT = {"seed": 8, "std": 0.02, "norm_std": 0.02, "page_size": 16}

# head_dim 128 with 4 query heads a KV head AND a window on the second and third layer (two cache
# groups): the window's edge, and the pages it gives back, through the tensor-core attention kernels
TINY_F = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 280,
    "hidden_size": 512,
    "intermediate_size": 272,
    "num_hidden_layers": 3,
    "num_attention_heads": 4,
    "num_key_value_heads": 1,
    "max_position_embeddings": 1024,
    "rope_theta": 500000.0,
    "rms_norm_eps": 1e-5,
    "attention_bias": True,
    "tie_word_embeddings": False,
    "use_sliding_window": True,
    "sliding_window": 150,
    "max_window_layers": 1,
}
TINY_F_INIT = {"seed": 9, "std": 0.02, "norm_std": 0.02, "page_size": 16}

# long contexts: head_dim 128 given by its own key (hidden / heads would be 48), two query heads a KV
# head, positions up to 8,192
TINY_G = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 300,
    "hidden_size": 192,
    "head_dim": 128,
    "intermediate_size": 256,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "max_position_embeddings": 8192,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": True,
    "tie_word_embeddings": False,
}
TINY_G_INIT = {"seed": 10, "std": 0.03, "norm_std": 0.02, "page_size": 16}

ALL = {"G": (TINY_G, TINY_G_INIT), "F": (TINY_F, TINY_F_INIT), "A": (TINY_A, TINY_A_INIT), "B": (TINY_B, TINY_B_INIT), "C": (TINY_C, TINY_C_INIT), "D": (TINY_D, TINY_D_INIT),
       "E": (TINY_E, TINY_E_INIT)}


def head_dim(cfg: dict) -> int:
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def tensor_shapes(cfg: dict) -> list:
    """(name, shape, is_norm) of every checkpoint tensor, in a fixed order."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d = head_dim(cfg)
    q, kv = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d
    out = [("model.embed_tokens.weight", (V, H), False)]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out.append((p + "input_layernorm.weight", (H,), True))
        for name, rows in (("q_proj", q), ("k_proj", kv), ("v_proj", kv)):
            out.append((p + f"self_attn.{name}.weight", (rows, H), False))
            if cfg.get("attention_bias", True):
                out.append((p + f"self_attn.{name}.bias", (rows,), False))
        out.append((p + "self_attn.o_proj.weight", (H, q), False))
        out.append((p + "post_attention_layernorm.weight", (H,), True))
        out.append((p + "mlp.gate_proj.weight", (I, H), False))
        out.append((p + "mlp.up_proj.weight", (I, H), False))
        out.append((p + "mlp.down_proj.weight", (H, I), False))
    out.append(("model.norm.weight", (H,), True))
    if not cfg.get("tie_word_embeddings", False):
        out.append(("lm_head.weight", (V, H), False))
    return out


def make_weights(cfg: dict, seed: int, std: float, norm_std: float, dtype=torch.float32, **_) -> dict:
    """Random weights written by the tests themselves (not by the package)."""
    g = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape, is_norm in tensor_shapes(cfg):
        noise = torch.randn(shape, generator=g, dtype=torch.float32)
        weights[name] = (1.0 + noise * norm_std if is_norm else noise * std).to(dtype)
    return weights


def make_ids(cfg: dict, length: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab_size"], (length,), generator=g).tolist()


def write_model_dir(folder, cfg: dict, weights: dict):
    import json
    from pathlib import Path

    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder
