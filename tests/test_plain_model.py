"""The plain implementation against the reference's own CPU model code (golden file)
and against itself where the reference has nothing to compare with (window, schedule)."""
import pathlib

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs

GOLDEN = pathlib.Path(__file__).parent / "golden" / "reference_logits.npz"


def _golden_weights(golden, name):
    """The weights the golden logits were made with, stored as bfloat16 bit patterns."""
    prefix = f"{name}_weight:"
    out = {}
    for key in golden.files:
        if key.startswith(prefix):
            bits = torch.from_numpy(golden[key].astype(np.int32)) << 16
            out[key[len(prefix):]] = bits.view(torch.float32)
    return out


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_model_code(name):
    golden = np.load(GOLDEN)
    cfg, init = tiny_configs.ALL[name]
    cfg = {k: v for k, v in cfg.items() if k not in ("use_sliding_window", "sliding_window", "max_window_layers")}
    weights = _golden_weights(golden, name)
    assert {n for n, _, _ in tiny_configs.tensor_shapes(cfg)} == set(weights)
    ids = golden[f"{name}_ids"].tolist()
    logits = plain_model.forward_logits(cfg, weights, ids).numpy()
    np.testing.assert_allclose(logits, golden[f"{name}_dense"], rtol=0, atol=2e-6)
    # the reference's paged prefill + decode gives the same positions' logits
    np.testing.assert_allclose(logits[29:], golden[f"{name}_paged_from_30"], rtol=0, atol=5e-6)


def test_window_wider_than_sequence_changes_nothing():
    cfg, init = tiny_configs.ALL["B"]
    weights = tiny_configs.make_weights(cfg, **init)
    ids = tiny_configs.make_ids(cfg, 30, seed=3)
    no_window = {k: v for k, v in cfg.items() if k != "use_sliding_window"}
    a = plain_model.forward_logits(cfg, weights, ids)  # window 40 > 30 tokens
    b = plain_model.forward_logits(no_window, weights, ids)
    assert torch.equal(a, b)


def test_window_drops_far_keys():
    q = torch.zeros(6, 1, 4)
    k = torch.zeros(6, 1, 4)
    v = torch.arange(6, dtype=torch.float32).view(6, 1, 1).expand(6, 1, 4).contiguous()
    out = plain_model.causal_gqa_attention(q, k, v, window=2)
    # uniform weights over the last 2 positions: mean of (t-1, t)
    assert torch.allclose(out[:, 0], torch.tensor([0.0, 0.5, 1.5, 2.5, 3.5, 4.5]))
    full = plain_model.causal_gqa_attention(q, k, v)
    assert torch.allclose(full[:, 0], torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 2.5]))


def test_window_against_a_query_by_query_restatement():
    """The masked-matrix form of the plain attention against loops over queries and keys that
    spell the rule out: query t of head h sees the keys of KV head h // g at positions
    max(0, t - window + 1) .. t, i.e. ``window`` keys, itself included."""
    g = torch.Generator().manual_seed(5)
    T, nh, nkv, d, window = 23, 6, 2, 8, 5
    q, k, v = (torch.randn(T, n, d, generator=g) for n in (nh, nkv, nkv))
    got = plain_model.causal_gqa_attention(q, k, v, window=window).view(T, nh, d)
    for t in range(T):
        keys = list(range(max(0, t - window + 1), t + 1))
        assert len(keys) == min(window, t + 1)
        for h in range(nh):
            kv = h // (nh // nkv)
            scores = torch.tensor([float(q[t, h] @ k[j, kv]) / d ** 0.5 for j in keys], dtype=torch.float64)
            weights = torch.softmax(scores, dim=0)
            want = sum(w * v[j, kv].double() for w, j in zip(weights, keys))
            assert torch.allclose(got[t, h].double(), want, atol=1e-5)


def test_rope_keeps_norm_and_is_identity_at_zero():
    x = torch.randn(5, 3, 16, generator=torch.Generator().manual_seed(0))
    y = plain_model.rope_split_half(x, torch.arange(5), 10000.0)
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1), atol=1e-5)
    assert torch.allclose(x[0], y[0])


def test_schedule_with_repeated_layer_and_shared_cache_runs():
    cfg, init = tiny_configs.ALL["A"]
    weights = tiny_configs.make_weights(cfg, **init)
    ids = tiny_configs.make_ids(cfg, 12, seed=4)
    base = plain_model.forward_logits(cfg, weights, ids)
    twice = plain_model.forward_logits(cfg, weights, ids, schedule=[(0, None), (1, None), (0, None)])
    shared = plain_model.forward_logits(cfg, weights, ids, schedule=[(0, None), (1, 0)])
    assert base.shape == twice.shape == shared.shape
    assert not torch.allclose(base, twice) and not torch.allclose(base, shared)


def test_uniform_and_greedy():
    us = [plain_model.uniform_for(7, 3, i) for i in range(2000)]
    assert 0 < min(us) and max(us) < 1 and abs(sum(us) / len(us) - 0.5) < 0.03
    assert plain_model.uniform_for(7, 3, 5) != plain_model.uniform_for(7, 4, 5)
    assert int(plain_model.greedy(torch.tensor([1.0, 3.0, 3.0, 2.0]))) == 1
