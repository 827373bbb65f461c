"""Two more toy parts, defined HERE and registered without a change to the framework's files:
a feed-forward with ROUTING (each token goes to the one of three small experts that its router
score picks, weighted by the softmax of the scores) and ANOTHER POSITION ENCODING (a learned
vector per position added to the queries and keys, with a tensor of its own in the checkpoint).
They stand in layer 0 of a toy architecture beside an ordinary layer 1, so one model has two
kinds of feed-forward and two position encodings.  The toys are no model of anyone's; they
compute with ordinary tensor operations."""
import dataclasses
from dataclasses import dataclass

import pytest
import torch

import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu
EXPERTS = 3


def register_toys():
    from torchlet_b200.config import PartSpec, Qwen2Config, register_architecture
    from torchlet_b200.parts import FEED_FORWARDS, POSITIONS, FeedForward, Positions, TensorSpec

    @POSITIONS.register("toy_added_positions")
    class AddedPositions(Positions):
        """q += table[position], k += table[position] (every head the same vector).  It only
        encodes; the attention mixer stores k and v in the request's pages itself."""

        graph_safe = False  # indexes with host-side shapes: stays out of the captured decode graph

        def __init__(self, spec):
            super().__init__(spec)
            self.head_dim = int(spec.params["head_dim"])

        @classmethod
        def expected_tensors(cls, spec, prefix):
            return [TensorSpec(prefix + "position_table.weight", (int(spec.params["positions"]), int(spec.params["head_dim"])))]

        def load(self, tensors, prefix, device, dtype):
            self.table = tensors[prefix + "position_table.weight"].to(device=device, dtype=torch.float32)

        def encode(self, ctx, qkv, num_heads, num_kv_heads):
            d, T = self.head_dim, qkv.shape[0]
            add = self.table[ctx.positions.long()][:, None, :]
            q = qkv[:, : num_heads * d].view(T, num_heads, d)
            k = qkv[:, num_heads * d: (num_heads + num_kv_heads) * d].view(T, num_kv_heads, d)
            q.copy_((q.float() + add).to(qkv.dtype))
            k.copy_((k.float() + add).to(qkv.dtype))

    @FEED_FORWARDS.register("toy_switch")
    class SwitchFeedForward(FeedForward):
        """acc += p_e(x) * W_e x for the expert e = argmax of the router scores; p = softmax."""

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden = int(spec.params["hidden_size"])
            self.experts = int(spec.params["experts"])

        @classmethod
        def expected_tensors(cls, spec, prefix):
            h, e = int(spec.params["hidden_size"]), int(spec.params["experts"])
            return [TensorSpec(prefix + "router.weight", (e, h))] + [
                TensorSpec(f"{prefix}experts.{i}.weight", (h, h)) for i in range(e)]

        def load(self, tensors, prefix, device, dtype):
            self.router = tensors[prefix + "router.weight"].to(device=device, dtype=torch.float32)
            self.weights = [tensors[f"{prefix}experts.{i}.weight"].to(device=device, dtype=torch.float32)
                            for i in range(self.experts)]

        def forward(self, ctx, x, acc):
            x = x.float()
            scores = x @ self.router.t()  # router logits in float32
            chosen = scores.argmax(dim=-1)
            weight = torch.softmax(scores, dim=-1).gather(1, chosen[:, None])
            for e in range(self.experts):
                rows = (chosen == e).nonzero().flatten()
                if rows.numel():
                    acc[rows] += weight[rows] * (x[rows] @ self.weights[e].t())

    @register_architecture("ToyPartsForCausalLM")
    @dataclass(frozen=True)
    class ToyConfig:
        base: Qwen2Config

        @classmethod
        def from_dict(cls, raw):
            return cls(Qwen2Config.from_dict(dict(raw, architectures=["Qwen2ForCausalLM"])))

        def to_dict(self):
            return dict(self.base.to_dict(), architectures=["ToyPartsForCausalLM"])

        def __getattr__(self, name):
            return getattr(self.base, name)

        def model_spec(self):
            spec = self.base.model_spec()
            first = spec.layers[0]
            positions = PartSpec("toy_added_positions", {"head_dim": self.base.head_dim,
                                                         "positions": self.base.max_position_embeddings})
            mixer = PartSpec(first.mixer.kind, dict(first.mixer.params, positions=positions))
            switch = PartSpec("toy_switch", {"hidden_size": self.base.hidden_size, "experts": EXPERTS})
            layers = (dataclasses.replace(first, mixer=mixer, feed_forward=switch),) + tuple(spec.layers[1:])
            return dataclasses.replace(spec, architecture="ToyPartsForCausalLM", layers=layers)

    return ToyConfig


def plain_toy_logits(cfg, w, ids):
    """Whole sequence, no cache: layer 0 with the added positions and the routed feed-forward,
    layer 1 as usual."""
    eps = cfg["rms_norm_eps"]
    T = len(ids)
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg["hidden_size"] // nh
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    h = plain_model.rms_norm(x, w["model.layers.0.input_layernorm.weight"], eps)
    p = "model.layers.0.self_attn."
    add = w[p + "position_table.weight"][:T][:, None, :]
    q = plain_model.linear(h, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).view(T, nh, d) + add
    k = plain_model.linear(h, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(T, nkv, d) + add
    v = plain_model.linear(h, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(T, nkv, d)
    x = x + plain_model.linear(plain_model.causal_gqa_attention(q, k, v), w[p + "o_proj.weight"])
    h = plain_model.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], eps)
    scores = h @ w["model.layers.0.mlp.router.weight"].t()
    chosen = scores.argmax(dim=-1)
    weight = torch.softmax(scores, dim=-1).gather(1, chosen[:, None])
    experts = torch.stack([w[f"model.layers.0.mlp.experts.{e}.weight"] for e in range(EXPERTS)])
    x = x + weight * torch.einsum("th,toh->to", h, experts[chosen])
    x, _ = plain_model.transformer_block(x, w, "model.layers.1.", cfg, None)
    x = plain_model.rms_norm(x, w["model.norm.weight"], eps)
    return x @ w["model.embed_tokens.weight"].t(), chosen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(tmp_path, dtype):
    from torchlet_b200.config import EngineConfig, known_architectures
    from torchlet_b200.engine import ModelRunner, StepEntry
    from torchlet_b200.engine.loading import load_model
    from torchlet_b200.weights import read_safetensors, write_random_model

    ToyConfig = register_toys()
    assert "ToyPartsForCausalLM" in known_architectures()
    raw = dict(tiny_configs.TINY_A, architectures=["ToyPartsForCausalLM"], max_position_embeddings=96)
    config = ToyConfig.from_dict(raw)
    folder = write_random_model(tmp_path / "toy", config, seed=9, std=0.05, norm_std=0.02)
    names = set(read_safetensors(folder))
    assert "model.layers.0.self_attn.position_table.weight" in names  # the encoding's own tensor
    assert "model.layers.0.mlp.router.weight" in names and "model.layers.1.mlp.gate_proj.weight" in names
    model = load_model(folder, dtype)
    assert type(model.blocks[0].feed_forward).__name__ == "SwitchFeedForward"
    assert type(model.blocks[1].feed_forward).__name__ != "SwitchFeedForward"
    assert type(model.blocks[0].mixer.positions).__name__ == "AddedPositions"
    assert not model.blocks[0].mixer.graph_safe and model.blocks[1].mixer.graph_safe
    runner = ModelRunner(model, EngineConfig(dtype=dtype, max_decode_slots=2, kv_block_size=16, max_seq_len=96,
                                             max_num_blocks=14))

    w = {k: v.float() for k, v in read_safetensors(folder).items()}
    seqs = [tiny_configs.make_ids(raw, n, seed=40 + i) for i, n in enumerate((47, 30))]
    plain = [plain_toy_logits(raw, w, ids) for ids in seqs]
    assert all(len(set(chosen.tolist())) > 1 for _, chosen in plain), "the router never switched"
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    # the two requests in portions, beside each other, then token by token
    got = {0: [], 1: []}
    runner.admit("r0"); runner.admit("r1")
    plan = [[(0, 0, 20), (1, 0, 3)], [(0, 20, 2), (1, 3, 25)], [(0, 22, 24), (1, 28, 1)], [(0, 46, 1), (1, 29, 1)]]
    for step in plan:
        logits = runner.step([StepEntry(f"r{r}", seqs[r][a:a + n], list(range(n))) for r, a, n in step]).cpu()
        row = 0
        for r, a, n in step:
            got[r].append(logits[row:row + n].clone())
            row += n
    assert runner.graph_steps == 0  # the toy position encoding keeps the model out of the decode graph
    for r in range(2):
        out, want = torch.cat(got[r]), plain[r][0]
        # (with these seeds no router score is so close to a tie that bfloat16 rounding flips the choice)
        assert (out - want).abs().max() <= tol * want.abs().max(), f"request {r}"
    runner.finish("r0"); runner.finish("r1")
    runner.cache.check()
