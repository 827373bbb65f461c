"""Each part of a layer alone against its plain function, at sizes of their own, driven
through a real step context (so positions, block tables and pages are the engine's)."""
import pytest
import torch

import harness
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def context(runner, lens_before, q_lens, seed=0):
    """Admit requests, give them ``lens_before`` cached tokens by stepping random ids, then
    build (without running) a step of ``q_lens`` new tokens each; returns ctx, caches."""
    from torchlet_b200.engine import StepEntry

    cfg = runner.model.config
    ids = []
    for i, (before, q) in enumerate(zip(lens_before, q_lens)):
        runner.admit(f"p{i}")
        tokens = tiny_configs.make_ids({"vocab_size": cfg.vocab_size}, before + q, seed + i)
        ids.append(tokens)
        if before:
            runner.step([StepEntry(f"p{i}", tokens[:before])])
    entries = [StepEntry(f"p{i}", ids[i][before:]) for i, before in enumerate(lens_before)]
    return runner._build(entries), ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import NORMS, build_part

    runner = harness.make_runner("A", dtype)
    (ctx, _), _ = context(runner, [0], [9])
    norm = build_part(NORMS, PartSpec("rms_norm", {"size": 100, "eps": 3e-5}))
    weight = torch.randn(100) * 0.1 + 1
    norm.load({"n.weight": weight.to(torch.bfloat16)}, "n.", DEV, runner.dtype)
    acc = torch.randn(9, 100, device=DEV) * 2
    out = norm.forward(ctx, acc)
    want = plain_model.rms_norm(acc.cpu(), weight.to(torch.bfloat16).float(), 3e-5)
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert out.dtype == runner.dtype and (out.float().cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_attention_mixer_part(name, dtype):
    """The mixer of layer 0 alone: projections, rotary, cache write, attention over cached
    context plus new tokens, output projection added into the stream."""
    runner = harness.make_runner(name, dtype, num_pages=64)
    cfg, w = harness.weights_for(name)
    lens_before, q_lens = [20, 0, 37], [5, 33, 1]
    (ctx, caches), ids = context(runner, lens_before, q_lens)
    mixer = runner.model.blocks[0].mixer
    hidden = cfg["hidden_size"]
    g = torch.Generator().manual_seed(3)
    # the mixer's input for ALL tokens of each request (cached and new): the cached part must
    # be what earlier steps fed, so recompute it the plain way: x = norm(embedding)
    table = w["model.embed_tokens.weight"]
    eps = cfg["rms_norm_eps"]
    outs, rows = [], []
    for i, (before, q) in enumerate(zip(lens_before, q_lens)):
        x_all = plain_model.rms_norm(table[torch.tensor(ids[i])], w["model.layers.0.input_layernorm.weight"], eps)
        y, _ = plain_model.attention_mixer(x_all, w, "model.layers.0.", cfg, plain_model.layer_window(cfg, 0))
        outs.append(y[before:])
        rows.append(x_all[before:])
    x = torch.cat(rows).to(DEV).to(runner.dtype)
    acc = torch.zeros(sum(q_lens), hidden, device=DEV)
    mixer.forward(ctx, x, acc, caches[0])
    ctx.flush_pending()
    want = torch.cat(outs)
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    assert (acc.cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_feed_forward_part(name, dtype):
    runner = harness.make_runner(name, dtype)
    cfg, w = harness.weights_for(name)
    (ctx, _), _ = context(runner, [0, 0], [7, 300])
    ffn = runner.model.blocks[1].feed_forward
    x = (torch.randn(307, cfg["hidden_size"], generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    base = torch.randn(307, cfg["hidden_size"], generator=torch.Generator().manual_seed(2))
    acc = base.clone().to(DEV)
    ffn.forward(ctx, x.to(DEV).to(runner.dtype), acc)
    ctx.flush_pending()
    want = base + plain_model.swiglu_feed_forward(x.float(), w, "model.layers.1.")
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    assert (acc.cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part(dtype):
    runner = harness.make_runner("B", dtype)
    cfg, w = harness.weights_for("B")
    (ctx, caches), ids = context(runner, [0], [50])
    x0 = w["model.embed_tokens.weight"][torch.tensor(ids[0])]
    acc = x0.clone().to(DEV)
    runner.model.blocks[0].forward(ctx, acc, caches[0])
    ctx.flush_pending()
    want, _ = plain_model.transformer_block(x0, w, "model.layers.0.", cfg, plain_model.layer_window(cfg, 0))
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert (acc.cpu() - want).abs().max() <= tol * want.abs().max()


def test_parts_are_chosen_layer_by_layer():
    """Tiny B: layer 0 sees all keys, layers 1 and 2 a window; two cache groups result."""
    runner = harness.make_runner("B", "float32")
    windows = [block.mixer.window for block in runner.model.blocks]
    assert windows == [None, 40, 40]
    assert [(g.window, g.entries) for g in runner.storage.groups] == [(None, (0,)), (40, (1, 2))]
    assert runner.storage.pages[0].shape[0] == 1 and runner.storage.pages[1].shape[0] == 2
