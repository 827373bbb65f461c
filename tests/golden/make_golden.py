"""Makes tests/golden/reference_logits.npz: logits of the REFERENCE's own model code
(4mengy/torchlet, CPU, float32) on tiny random models, against which the plain
implementation in tests/plain_model.py is checked once.

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

Uses torchlet.v00_full_recompute (dense whole-sequence forward) and
torchlet.v08_paged_gqa_py (paged prefill of a prefix, then paged decode token by
token) — the versions whose forward runs on the CPU.  The reference has no window, so
tiny B is used with its window keys removed.  Stored: token ids, a checksum of the
weights (drawn by tests/tiny_configs.make_weights) and the logits.
"""
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import tiny_configs  # noqa: E402


def dense_logits(cfg, weights, ids):
    from torchlet.v00_full_recompute.model.qwen2_5 import Qwen2ForCausalLM

    model = Qwen2ForCausalLM(cfg)
    missing = model.load_state_dict(weights, strict=False)
    assert not missing.unexpected_keys, missing
    model.eval()
    with torch.no_grad():
        return model(torch.tensor([ids]))[0]


def paged_logits(cfg, weights, ids, prefill, block_size=8):
    """v08: paged prefill of ids[:prefill] (last-token logits), then one decode step per
    remaining token; returns logits for positions prefill-1 .. len(ids)-1."""
    from torchlet.v08_paged_gqa_py.forward_params import ForwardParams
    from torchlet.v08_paged_gqa_py.kvcache import KVCache
    from torchlet.v08_paged_gqa_py.model.qwen2_5 import Qwen2ForCausalLM

    model = Qwen2ForCausalLM(cfg)
    model.load_state_dict(weights, strict=False)
    model.eval()
    slots, max_seq = 2, cfg["max_position_embeddings"]
    per_req = -(-max_seq // block_size)
    d = tiny_configs.head_dim(cfg)
    cache = KVCache(cfg["num_hidden_layers"], slots * per_req + 1, slots, block_size,
                    cfg["num_key_value_heads"], max_seq, d, "cpu", torch.float32)
    table = torch.zeros(slots, per_req, dtype=torch.long)
    pages = list(range(3, 3 + -(-len(ids) // block_size)))[::-1]  # an odd order on purpose
    table[1, :len(pages)] = torch.tensor(pages)
    out = []
    with torch.no_grad():
        fp = ForwardParams(torch.tensor([0, prefill]), torch.arange(prefill), [1], None, True, cache, table)
        out.append(model(torch.tensor(ids[:prefill]), fp, last_token_only=True)[0])
        for pos in range(prefill, len(ids)):
            tokens = torch.zeros(slots, dtype=torch.long)
            tokens[1] = ids[pos]
            positions = torch.zeros(slots, dtype=torch.long)
            positions[1] = pos
            active = torch.tensor([False, True])
            fp = ForwardParams(torch.arange(slots + 1), positions, None, active, False, cache, table)
            out.append(model(tokens, fp)[1])
    return torch.stack(out)


def main():
    store = {}
    for name in ("A", "B"):
        cfg, init = tiny_configs.ALL[name]
        cfg = {k: v for k, v in cfg.items() if k not in ("use_sliding_window", "sliding_window", "max_window_layers")}
        weights = {k: v.float() for k, v in tiny_configs.make_weights(cfg, dtype=torch.bfloat16, **init).items()}
        ids = tiny_configs.make_ids(cfg, 45, seed=11)
        store[f"{name}_ids"] = np.array(ids, dtype=np.int64)
        for key, value in weights.items():  # bfloat16-representable: the upper 16 bits say it all
            store[f"{name}_weight:{key}"] = (value.contiguous().view(torch.int32) >> 16).to(torch.int16).numpy()
        store[f"{name}_dense"] = dense_logits(cfg, weights, ids).numpy()
        store[f"{name}_paged_from_30"] = paged_logits(cfg, weights, ids, 30).numpy()
    np.savez_compressed(HERE / "reference_logits.npz", **store)
    for key, value in store.items():
        if "_weight:" not in key:
            print(key, value.shape)


if __name__ == "__main__":
    main()
