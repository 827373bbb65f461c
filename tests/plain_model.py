"""Plain, slow implementation of the model: whole sequences, no cache, float32 by
default, one function for each part.  It shares no code with ``torchlet_b200`` and is
written from the reference's formulas; each function cites the file and lines it
restates (paths are relative to the reference project's ``src/torchlet``).

It was compared once with the reference's own CPU model code on tiny random models;
``tests/golden/make_golden.py`` is the script and ``tests/golden/*.npz`` its output.

Weights are a dict of tensor name -> torch tensor, with the checkpoint's names.
A configuration is a plain dict with config.json's keys.
"""
from __future__ import annotations

import math

import torch


def cfg_get(cfg: dict, key: str, default=None):
    value = cfg.get(key, default)
    return default if value is None else value


def rope_theta(cfg: dict) -> float:
    """v10_triton_paged_gqa/model/qwen2_5.py:14-18."""
    rope_parameters = cfg.get("rope_parameters")
    if isinstance(rope_parameters, dict) and "rope_theta" in rope_parameters:
        return float(rope_parameters["rope_theta"])
    return float(cfg_get(cfg, "rope_theta", 1_000_000.0))


def head_dim(cfg: dict) -> int:
    """v00_full_recompute/layer/gqa.py:30 (hidden // heads); a ``head_dim`` key wins."""
    return int(cfg_get(cfg, "head_dim", cfg["hidden_size"] // cfg["num_attention_heads"]))


def layer_window(cfg: dict, layer: int):
    """Window of a layer, from the sliding-window keys (the reference ignores them):
    on for layers at or past ``max_window_layers`` when ``use_sliding_window``."""
    if cfg_get(cfg, "use_sliding_window", False) and layer >= cfg_get(cfg, "max_window_layers", 0):
        return int(cfg["sliding_window"])
    return None


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """v10_triton_paged_gqa/model/qwen2_5.py:56."""
    return table[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """v08_paged_gqa_py/layer/rms_norm.py:11-14: x * rsqrt(mean(x^2) + eps) * w."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def linear(x: torch.Tensor, weight: torch.Tensor, bias=None) -> torch.Tensor:
    """nn.Linear layout [out, in], y = x W^T + b (v00_full_recompute/layer/gqa.py:33-38)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def rope_angles(positions: torch.Tensor, dim: int, theta: float) -> torch.Tensor:
    """v08_paged_gqa_py/layer/rope.py:29-35: inv_freq_i = 1 / theta^(2i/d) in float32,
    angle[p, i] = p * inv_freq_i in float32."""
    i = torch.arange(0, dim, 2, dtype=torch.float32)
    inv_freq = 1.0 / (theta ** (i / dim))
    return torch.outer(positions.to(torch.float32), inv_freq)


def rope_split_half(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """v08_paged_gqa_py/layer/rope.py:46-66: y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin
    with x1/x2 the first/second half of the head.  x: [T, heads, d]."""
    d = x.shape[-1]
    angles = rope_angles(positions, d, theta)  # [T, d/2]
    cos = angles.cos().to(x.dtype)[:, None, :]
    sin = angles.sin().to(x.dtype)[:, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2 :]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def causal_gqa_attention(q, k, v, window=None, scale=None) -> torch.Tensor:
    """v00_full_recompute/layer/gqa.py:63-88: query head h reads KV head h // g
    (repeat_interleave), scores q.k, future positions -inf, softmax(scores / sqrt(d)),
    weights @ values.  ``window``: a key is also dropped when it lies ``window`` or
    more positions behind the query.  q: [T, nh, d]; k, v: [T, nkv, d] -> [T, nh*d]."""
    T, nh, d = q.shape
    g = nh // k.shape[1]
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, kk)
    pos = torch.arange(T)
    dropped = pos[None, :] > pos[:, None]
    if window is not None:
        dropped = dropped | (pos[:, None] - pos[None, :] >= window)
    scores = scores.masked_fill(dropped[None], float("-inf"))
    factor = (1.0 / math.sqrt(d)) if scale is None else scale
    weights = torch.softmax(scores * factor, dim=-1)
    out = torch.einsum("hqk,khd->qhd", weights, vv)
    return out.reshape(T, nh * d)


def attention_mixer(x, w: dict, prefix: str, cfg: dict, window, positions=None, kv_override=None):
    """v00_full_recompute/layer/gqa.py:43-91 (projections, heads, RoPE on q and k,
    attention, unbiased output projection).  Returns (output, (k, v)) so that another
    execution can read this one's keys and values."""
    T = x.shape[0]
    nh = cfg["num_attention_heads"]
    nkv = cfg_get(cfg, "num_key_value_heads", nh)
    d = head_dim(cfg)
    theta = rope_theta(cfg)
    if positions is None:
        positions = torch.arange(T)
    p = prefix + "self_attn."
    q = linear(x, w[p + "q_proj.weight"], w.get(p + "q_proj.bias")).view(T, nh, d)
    q = rope_split_half(q, positions, theta)
    if kv_override is None:
        k = linear(x, w[p + "k_proj.weight"], w.get(p + "k_proj.bias")).view(T, nkv, d)
        v = linear(x, w[p + "v_proj.weight"], w.get(p + "v_proj.bias")).view(T, nkv, d)
        k = rope_split_half(k, positions, theta)
    else:
        k, v = kv_override
    ctx = causal_gqa_attention(q, k, v, window)
    return linear(ctx, w[p + "o_proj.weight"]), (k, v)


def swiglu_feed_forward(x, w: dict, prefix: str) -> torch.Tensor:
    """v08_paged_gqa_py/layer/ffn_swiglu.py:12-15: down(silu(gate(x)) * up(x))."""
    p = prefix + "mlp."
    gate = linear(x, w[p + "gate_proj.weight"])
    up = linear(x, w[p + "up_proj.weight"])
    return linear(torch.nn.functional.silu(gate) * up, w[p + "down_proj.weight"])


def transformer_block(x, w: dict, prefix: str, cfg: dict, window, kv_override=None):
    """v00_full_recompute/layer/transformer_block.py:36-39: pre-norm residual."""
    eps = float(cfg_get(cfg, "rms_norm_eps", 1e-6))
    attn, kv = attention_mixer(
        rms_norm(x, w[prefix + "input_layernorm.weight"], eps), w, prefix, cfg, window, kv_override=kv_override
    )
    x = x + attn
    x = x + swiglu_feed_forward(rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps), w, prefix)
    return x, kv


def forward_logits(cfg: dict, weights: dict, ids, schedule=None, dtype=torch.float32) -> torch.Tensor:
    """v10_triton_paged_gqa/model/qwen2_5.py:55-60, 82-87: embedding, the layers, final
    norm, LM head (tied to the embedding when ``tie_word_embeddings``).  Logits of every
    position of ONE sequence, [T, vocab].  ``schedule``: list of (layer, cache_from)
    pairs; default each layer once in order."""
    w = {name: t.to(dtype) if t.is_floating_point() else t for name, t in weights.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    n_layers = cfg["num_hidden_layers"]
    if schedule is None:
        schedule = [(i, None) for i in range(n_layers)]
    x = embedding(ids, w["model.embed_tokens.weight"])
    kvs = []
    for layer, cache_from in schedule:
        kv_override = None if cache_from is None else kvs[cache_from]
        x, kv = transformer_block(x, w, f"model.layers.{layer}.", cfg, layer_window(cfg, layer), kv_override)
        kvs.append(kv)
    x = rms_norm(x, w["model.norm.weight"], float(cfg_get(cfg, "rms_norm_eps", 1e-6)))
    head = w["model.embed_tokens.weight"] if cfg_get(cfg, "tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, head)


# --------------------------------------------------------------------- sampling
def greedy(logits: torch.Tensor) -> torch.Tensor:
    """v10_triton_paged_gqa/engine.py:187-188: argmax; the lowest index wins a tie."""
    return torch.argmax(logits, dim=-1)


_MASK64 = (1 << 64) - 1


def _mix64(x: int) -> int:
    x &= _MASK64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _MASK64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _MASK64
    x ^= x >> 31
    return x


def uniform_for(seed: int, counter: int, index: int) -> float:
    """The engine's counter-based uniform in (0, 1): two rounds of a 64-bit mixer over
    (seed, counter) then the vocabulary index; the top 23 bits give the fraction.
    (The reference samples greedily only; this restates the engine's documented draw.)"""
    key = _mix64((seed & _MASK64) * 0x9E3779B97F4A7C15 + (counter & _MASK64) + 0x632BE59BD9B4E019)
    bits = _mix64(key ^ ((index + 1) * 0xD1B54A32D192ED03 & _MASK64))
    return ((bits >> 41) + 0.5) / float(1 << 23)


def temperature_scores(logits, temperature: float, seed: int, counter: int):
    """Scores whose argmax is a draw from softmax(logits / temperature): logits / T plus
    Gumbel noise -log(-log(u)) with u from ``uniform_for``.  float64 list, one row."""
    out = []
    for i, value in enumerate(logits.tolist()):
        u = uniform_for(seed, counter, i)
        out.append(value / temperature - math.log(-math.log(u)))
    return out


def greedy_generate(cfg, weights, prompt, max_new_tokens, schedule=None, dtype=torch.float32):
    """v00_full_recompute/llm.py:47-87: recompute the whole sequence for every token."""
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        logits = forward_logits(cfg, weights, ids, schedule, dtype)
        token = int(greedy(logits[-1]))
        out.append(token)
        ids.append(token)
    return out
