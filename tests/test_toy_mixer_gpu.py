"""A toy mixer with state of its own, defined HERE, is registered, built and stepped
without a change to the framework's files: a running mean of its inputs per request,
kept in the request's slot between steps.  It stands in one layer of a toy architecture
(registered here too) beside an ordinary attention layer, so the model has different
mixers in different layers.  The toy is no model of anyone's."""
from dataclasses import dataclass

import pytest
import torch

import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def register_toy():
    from torchlet_b200.config import LayerSpec, ModelSpec, PartSpec, Qwen2Config, ScheduleEntry, register_architecture
    from torchlet_b200.parts import MIXERS, Mixer, StateSpec, TensorSpec

    @MIXERS.register("toy_running_mean")
    class RunningMeanMixer(Mixer):
        """y_t = W . mean(x_0 .. x_t); the sum so far is the per-request state."""

        graph_safe = False  # plans on the host: keeps out of the captured decode graph

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

    @register_architecture("ToyStateForCausalLM")
    @dataclass(frozen=True)
    class ToyConfig:
        base: Qwen2Config

        @classmethod
        def from_dict(cls, raw):
            return cls(Qwen2Config.from_dict(dict(raw, architectures=["Qwen2ForCausalLM"])))

        def to_dict(self):
            return dict(self.base.to_dict(), architectures=["ToyStateForCausalLM"])

        def __getattr__(self, name):
            return getattr(self.base, name)

        def model_spec(self):
            import dataclasses

            spec = self.base.model_spec()
            toy = PartSpec("toy_running_mean", {"hidden_size": self.base.hidden_size})
            layers = list(spec.layers)
            layers[0] = dataclasses.replace(layers[0], mixer=toy)
            return dataclasses.replace(spec, architecture="ToyStateForCausalLM", layers=tuple(layers))

    return ToyConfig


def plain_toy_logits(cfg, w, ids):
    """Whole sequence, no state: layer 0 with the running-mean mixer, layer 1 as usual."""
    eps = cfg["rms_norm_eps"]
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    h = plain_model.rms_norm(x, w["model.layers.0.input_layernorm.weight"], eps)
    means = torch.cumsum(h, dim=0) / torch.arange(1, len(ids) + 1).unsqueeze(1)
    x = x + means @ w["model.layers.0.self_attn.mix.weight"].t()
    x = x + plain_model.swiglu_feed_forward(
        plain_model.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], eps), w, "model.layers.0.")
    x, _ = plain_model.transformer_block(x, w, "model.layers.1.", cfg, None)
    x = plain_model.rms_norm(x, w["model.norm.weight"], eps)
    return x @ w["model.embed_tokens.weight"].t()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    from torchlet_b200.config import EngineConfig, known_architectures
    from torchlet_b200.engine import ModelRunner, StepEntry
    from torchlet_b200.engine.loading import load_model
    from torchlet_b200.weights import read_safetensors, write_random_model

    ToyConfig = register_toy()
    assert "ToyStateForCausalLM" in known_architectures()
    raw = dict(tiny_configs.TINY_A, architectures=["ToyStateForCausalLM"])
    config = ToyConfig.from_dict(raw)
    folder = write_random_model(tmp_path / "toy", config, seed=3, std=0.05, norm_std=0.02)  # random-weights mode
    model = load_model(folder, dtype)  # chosen through the registry by config.json
    assert type(model.blocks[0].mixer).__name__ == "RunningMeanMixer"
    assert type(model.blocks[1].mixer).__name__ == "AttentionMixer"
    runner = ModelRunner(model, EngineConfig(dtype=dtype, max_decode_slots=2, kv_block_size=16, max_seq_len=128,
                                             max_num_blocks=20))
    assert list(runner.storage.states) == [0] and runner.storage.states[0].shape == (2, 64)
    assert len(runner.storage.groups) == 1 and runner.storage.groups[0].entries == (1,)  # only layer 1 has pages

    w = {k: v.float() for k, v in read_safetensors(folder).items()}
    seqs = [tiny_configs.make_ids(raw, n, seed=20 + i) for i, n in enumerate((40, 23, 31))]
    want = [plain_toy_logits(raw, w, ids) for ids in seqs]
    tol = 2e-5 if dtype == "float32" else 2.5e-2

    # requests 0 and 1 interleaved in portions; request 2 then reuses a slot, whose state
    # must start from zero again
    got = {0: [], 1: [], 2: []}
    runner.admit("t0"); runner.admit("t1")
    plan = [[(0, 0, 7), (1, 0, 2)], [(0, 7, 1), (1, 2, 20)], [(0, 8, 30)], [(0, 38, 2), (1, 22, 1)]]
    for step in plan:
        entries = [StepEntry(f"t{r}", seqs[r][a:a + n], list(range(n))) for r, a, n in step]
        logits = runner.step(entries).cpu()
        row = 0
        for r, a, n in step:
            got[r].append(logits[row:row + n].clone())
            row += n
    runner.finish("t0"); runner.finish("t1")
    runner.admit("t2")
    for a, n in ((0, 30), (30, 1)):
        got[2].append(runner.step([StepEntry("t2", seqs[2][a:a + n], list(range(n)))]).cpu().clone())
    assert runner.graph_steps == 0  # the toy keeps the model out of the decode graph
    for r in range(3):
        out = torch.cat(got[r])
        assert (out - want[r]).abs().max() <= tol * want[r].abs().max(), f"request {r}"
