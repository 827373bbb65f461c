"""More toys, defined HERE, registered without a change to the framework's files:

* a toy architecture whose checkpoint names its tensors differently (``h.<i>.attn.``,
  ``h.<i>.ffn.``, ``h.<i>.ln_*.``, ``wte.weight``, ``ln_f.``), with two block arrangements of
  its own: a PARALLEL block with one shared norm, and a SANDWICH block with three norms (one
  of them after the mixer); a norm of its own (mean-subtracting, with a bias tensor) written
  with ordinary tensor operations and no knowledge of how products hand over their sums; and an
  attention mixer WITHOUT any position encoding;
* a toy model whose EVERY mixer keeps only fixed-size state (no page pool at all), driven
  through the scheduler with more requests than slots and a preemption.

The toys are no model of anyone's."""
import dataclasses
from dataclasses import dataclass

import pytest
import torch

import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu


def register_toys():
    from torchlet_b200.config import LayerSpec, ModelSpec, NormSlot, PartSpec, Qwen2Config, register_architecture
    from torchlet_b200.parts import BLOCKS, MIXERS, NORMS, Block, Mixer, Norm, StateSpec, TensorSpec

    @NORMS.register("toy_centered_norm")
    class CenteredNorm(Norm):
        """y = (x - mean) / sqrt(var + eps) * w + b.  Only ``forward``: the base class has already
        completed whatever sum into ``acc`` was unfinished."""

        def __init__(self, spec):
            super().__init__(spec)
            self.size, self.eps = int(spec.params["size"]), float(spec.params["eps"])

        @classmethod
        def expected_tensors(cls, spec, prefix):
            n = int(spec.params["size"])
            return [TensorSpec(prefix + "weight", (n,), init="ones"), TensorSpec(prefix + "bias", (n,))]

        def load(self, tensors, prefix, device, dtype):
            self.weight = tensors[prefix + "weight"].to(device=device, dtype=torch.float32)
            self.bias = tensors[prefix + "bias"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, acc, out=None, rows=None, name="normed"):
            x = acc if rows is None else acc[rows.long()]
            y = torch.nn.functional.layer_norm(x, (self.size,), self.weight, self.bias, self.eps)
            if out is None:
                out = ctx.buffer(name, tuple(y.shape), ctx.dtype)
            out.copy_(y)
            return out

    @BLOCKS.register("toy_parallel")
    class ParallelBlock(Block):
        """x' = x + mixer(n) + feed_forward(n), n = norm(x)."""

        norm_roles = ("shared",)

        def forward(self, ctx, acc, cache):
            n = self.norms["shared"].apply(ctx, acc, name="toy.shared")
            self.mixer.forward(ctx, n, acc, cache)
            self.feed_forward.forward(ctx, n, acc)

    @BLOCKS.register("toy_sandwich")
    class SandwichBlock(Block):
        """x = x + post(mixer(pre(x))); x = x + feed_forward(ff(x)): the mixer's output is normed
        before it joins the stream, so the mixer adds into a zeroed stream of its own."""

        norm_roles = ("pre", "post", "ff")

        def forward(self, ctx, acc, cache):
            x = self.norms["pre"].apply(ctx, acc)
            own = ctx.buffer("toy.own_stream", tuple(acc.shape), torch.float32)
            own.zero_()
            self.mixer.forward(ctx, x, own, cache)
            y = self.norms["post"].apply(ctx, own, name="toy.post")
            ctx.flush_pending()
            acc += y.float()
            x = self.norms["ff"].apply(ctx, acc)
            self.feed_forward.forward(ctx, x, acc)

    @MIXERS.register("toy_running_sum")
    class RunningSumMixer(Mixer):
        """y_t = W . (x_0 + ... + x_t) / (t + 1); the sum so far is the per-request state."""

        graph_safe = False

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden = int(spec.params["hidden_size"])

        def state_spec(self):
            return StateSpec((self.hidden,), "float32")

        @classmethod
        def expected_tensors(cls, spec, prefix):
            h = int(spec.params["hidden_size"])
            return [TensorSpec(prefix + "mix.weight", (h, h))]

        def load(self, tensors, prefix, device, dtype):
            self.weight = tensors[prefix + "mix.weight"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, x, acc, cache):
            indptr, slots = ctx.req_indptr_host, ctx.slots_host
            for i in range(ctx.num_requests):
                a, b, slot = int(indptr[i]), int(indptr[i + 1]), int(slots[i])
                sums = cache.state[slot] + torch.cumsum(x[a:b].float(), dim=0)
                counts = (ctx.positions[a:b] + 1).float().unsqueeze(1)
                acc[a:b] += (sums / counts) @ self.weight.t()
                cache.state[slot] = sums[-1]

    def renamed(base: Qwen2Config, architecture: str, layers) -> ModelSpec:
        spec = base.model_spec()
        return dataclasses.replace(spec, architecture=architecture, layers=tuple(layers), embedding_name="wte.weight",
                                   final_norm_prefix="ln_f.", lm_head_name="head.weight")

    class _Toy:
        architecture = ""

        @classmethod
        def from_dict(cls, raw):
            return cls(Qwen2Config.from_dict(dict(raw, architectures=["Qwen2ForCausalLM"])))

        def to_dict(self):
            return dict(self.base.to_dict(), architectures=[self.architecture])

        def __getattr__(self, name):
            return getattr(self.base, name)

    @register_architecture("ToyNamesForCausalLM")
    @dataclass(frozen=True)
    class ToyNamesConfig(_Toy):
        base: Qwen2Config
        architecture = "ToyNamesForCausalLM"

        def model_spec(self):
            first, second = self.base.model_spec().layers
            rms = first.norms[0].part
            centered = PartSpec("toy_centered_norm", {"size": self.base.hidden_size, "eps": 1e-5})
            bare = PartSpec("attention", dict(first.mixer.params, positions=None))  # no position encoding at all
            layers = [
                LayerSpec("h.0.", "toy_parallel", bare, first.feed_forward, norms=(NormSlot("shared", centered, "ln_1."),),
                          mixer_prefix="attn.", feed_forward_prefix="ffn."),
                LayerSpec("h.1.", "toy_sandwich", second.mixer, second.feed_forward,
                          norms=(NormSlot("pre", rms, "ln_1."), NormSlot("post", rms, "ln_post."),
                                 NormSlot("ff", centered, "ln_2.")),
                          mixer_prefix="attn.", feed_forward_prefix="ffn."),
            ]
            return renamed(self.base, self.architecture, layers)

    @register_architecture("ToyStateOnlyForCausalLM")
    @dataclass(frozen=True)
    class ToyStateOnlyConfig(_Toy):
        base: Qwen2Config
        architecture = "ToyStateOnlyForCausalLM"

        def model_spec(self):
            spec = self.base.model_spec()
            mixer = PartSpec("toy_running_sum", {"hidden_size": self.base.hidden_size})
            layers = [dataclasses.replace(layer, prefix=f"h.{i}.", mixer=mixer, mixer_prefix="mix.")
                      for i, layer in enumerate(spec.layers)]
            return renamed(self.base, self.architecture, layers)

    return ToyNamesConfig, ToyStateOnlyConfig


# ------------------------------------------------------------ plain restatements
def _attention(x, w, p, cfg, rotate: bool):
    T = x.shape[0]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg["hidden_size"] // nh
    q = plain_model.linear(x, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).view(T, nh, d)
    k = plain_model.linear(x, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(T, nkv, d)
    v = plain_model.linear(x, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(T, nkv, d)
    if rotate:
        pos = torch.arange(T)
        q = plain_model.rope_split_half(q, pos, cfg["rope_theta"])
        k = plain_model.rope_split_half(k, pos, cfg["rope_theta"])
    return plain_model.linear(plain_model.causal_gqa_attention(q, k, v), w[p + "o_proj.weight"])


def _swiglu(x, w, p):
    gate, up = plain_model.linear(x, w[p + "gate_proj.weight"]), plain_model.linear(x, w[p + "up_proj.weight"])
    return plain_model.linear(torch.nn.functional.silu(gate) * up, w[p + "down_proj.weight"])


def _centered(x, w, p):
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), w[p + "weight"], w[p + "bias"], 1e-5)


def plain_names_logits(cfg, w, ids):
    eps = cfg["rms_norm_eps"]
    x = w["wte.weight"][torch.tensor(ids)]
    n = _centered(x, w, "h.0.ln_1.")
    x = x + _attention(n, w, "h.0.attn.", cfg, rotate=False) + _swiglu(n, w, "h.0.ffn.")
    y = _attention(plain_model.rms_norm(x, w["h.1.ln_1.weight"], eps), w, "h.1.attn.", cfg, rotate=True)
    x = x + plain_model.rms_norm(y, w["h.1.ln_post.weight"], eps)
    x = x + _swiglu(_centered(x, w, "h.1.ln_2."), w, "h.1.ffn.")
    return plain_model.rms_norm(x, w["ln_f.weight"], eps) @ w["wte.weight"].t()


def plain_state_only_logits(cfg, w, ids):
    eps = cfg["rms_norm_eps"]
    x = w["wte.weight"][torch.tensor(ids)]
    counts = torch.arange(1, len(ids) + 1).unsqueeze(1)
    for i in range(cfg["num_hidden_layers"]):
        h = plain_model.rms_norm(x, w[f"h.{i}.input_layernorm.weight"], eps)
        x = x + (torch.cumsum(h, dim=0) / counts) @ w[f"h.{i}.mix.mix.weight"].t()
        x = x + _swiglu(plain_model.rms_norm(x, w[f"h.{i}.post_attention_layernorm.weight"], eps), w, f"h.{i}.mlp.")
    return plain_model.rms_norm(x, w["ln_f.weight"], eps) @ w["wte.weight"].t()


# ------------------------------------------------------------------------ tests
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_tensor_names_arrangements_norm_and_no_positions(tmp_path, dtype):
    from torchlet_b200.config import EngineConfig
    from torchlet_b200.engine import ModelRunner, StepEntry
    from torchlet_b200.engine.loading import load_model
    from torchlet_b200.weights import read_safetensors, write_random_model

    ToyNamesConfig, _ = register_toys()
    raw = dict(tiny_configs.TINY_A, architectures=["ToyNamesForCausalLM"])
    folder = write_random_model(tmp_path / "names", ToyNamesConfig.from_dict(raw), seed=13, std=0.05, norm_std=0.02)
    names = set(read_safetensors(folder))
    assert {"wte.weight", "h.0.ln_1.bias", "h.0.attn.q_proj.weight", "h.1.ln_post.weight", "h.1.ffn.down_proj.weight",
            "ln_f.weight"} <= names
    assert not any(part in n for n in names for part in ("self_attn", "mlp.", "layernorm", "model."))
    model = load_model(folder, dtype)
    assert model.blocks[0].mixer.positions is None and model.blocks[1].mixer.positions is not None
    assert sorted(model.blocks[1].norms) == ["ff", "post", "pre"]
    runner = ModelRunner(model, EngineConfig(dtype=dtype, max_decode_slots=2, kv_block_size=16, max_seq_len=128,
                                             max_num_blocks=14))
    w = {k: v.float() for k, v in read_safetensors(folder).items()}
    seqs = [tiny_configs.make_ids(raw, n, seed=60 + i) for i, n in enumerate((50, 37))]
    want = [plain_names_logits(raw, w, ids) for ids in seqs]
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    got = {0: [], 1: []}
    runner.admit("r0"); runner.admit("r1")
    plan = [[(0, 0, 21), (1, 0, 2)], [(0, 21, 1), (1, 2, 30)], [(0, 22, 27), (1, 32, 1)], [(0, 49, 1), (1, 33, 4)]]
    for step in plan:
        logits = runner.step([StepEntry(f"r{r}", seqs[r][a:a + n], list(range(n))) for r, a, n in step]).cpu()
        row = 0
        for r, a, n in step:
            got[r].append(logits[row:row + n].clone())
            row += n
    for r in range(2):
        out = torch.cat(got[r])
        worst = ((out - want[r]).abs().amax(dim=1) / want[r].abs().amax(dim=1)).max()
        assert worst <= tol, f"request {r}: {worst:.3e}"
    runner.finish("r0"); runner.finish("r1")
    runner.cache.check()


def test_a_model_whose_every_mixer_keeps_only_state(tmp_path):
    """No page pool exists.  Five requests on two slots through the engine's own loop, prompts
    cut by a small token budget, one request preempted in mid-flight and recomputed: the
    greedy outputs equal the plain implementation's."""
    from torchlet_b200.config import EngineConfig
    from torchlet_b200.engine.engine import Engine
    from torchlet_b200.engine.loading import load_model
    from torchlet_b200.engine.scheduler import Request
    from torchlet_b200.sampling import SamplingParams
    from torchlet_b200.weights import read_safetensors, write_random_model

    _, ToyStateOnlyConfig = register_toys()
    raw = dict(tiny_configs.TINY_A, architectures=["ToyStateOnlyForCausalLM"])
    folder = write_random_model(tmp_path / "state", ToyStateOnlyConfig.from_dict(raw), seed=17, std=0.05, norm_std=0.02)
    model = load_model(folder, "float32")
    engine = Engine(model, EngineConfig(dtype="float32", max_decode_slots=2, kv_block_size=16, max_seq_len=128,
                                        max_num_batched_tokens=24))
    runner = engine.runner
    assert runner.storage.groups == [] and runner.storage.pages == [] and sorted(runner.storage.states) == [0, 1]
    w = {k: v.float() for k, v in read_safetensors(folder).items()}
    prompts = [tiny_configs.make_ids(raw, n, seed=80 + i) for i, n in enumerate((31, 7, 40, 3, 18))]
    requests = [Request(p, SamplingParams(max_new_tokens=6)) for p in prompts]
    engine.add_requests(requests)
    steps = preempted = 0
    while engine.scheduler.has_work():
        engine.step()
        steps += 1
        if steps == 4 and len(engine.scheduler.running) == 2:
            engine.scheduler._preempt(engine.scheduler.running[-1])  # its slot's state is cleared on re-admission
            preempted += 1
        runner.cache.check()
        assert steps < 200
    assert preempted == 1 and engine.scheduler.stats.preemptions == 1
    assert runner.cache.num_free_slots == 2 and runner.cache.live_requests() == []
    for request, prompt in zip(requests, prompts):
        assert request.error is None
        ids = list(prompt)
        for token in request.output_tokens:
            logits = plain_state_only_logits(raw, w, ids)[-1]
            assert float(logits[token]) >= float(logits.max()) - 1e-5 * float(logits.abs().max())
            ids.append(token)
        assert len(request.output_tokens) == 6
