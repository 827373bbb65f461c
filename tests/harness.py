"""Helpers of the GPU tests: build an engine for a tiny configuration, replay token
sequences through the step function in different cuts, and the plain logits to compare
with.  Weights are rounded to bfloat16 once, so that the float32 and the bfloat16 engine
and the plain implementation all hold the same numbers."""
from __future__ import annotations

import functools

import torch

import plain_model
import tiny_configs

# Largest allowed |engine - plain| as a fraction of max |plain logits|.
# float32: summation order only.  bfloat16: activations are rounded to 8 bits of
# mantissa between kernels (2^-9 relative per rounding, a few dozen roundings deep).
TOLERANCE = {"float32": 2e-5, "bfloat16": 2.5e-2}


@functools.lru_cache(maxsize=None)
def weights_for(name: str):
    cfg, init = tiny_configs.ALL[name]
    w = tiny_configs.make_weights(cfg, dtype=torch.bfloat16, **init)
    return cfg, {k: v.float() for k, v in w.items()}


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int, schedule=None):
    cfg, w = weights_for(name)
    ids = tiny_configs.make_ids(cfg, length, seed)
    return ids, plain_model.forward_logits(cfg, w, ids, schedule=list(schedule) if schedule else None)


def make_runner(name: str, dtype: str, num_pages: int = 200, slots: int = 4, page_size=None, budget: int = 2048,
                schedule=None, max_seq_len=None, cuda_graph: bool = False):
    from torchlet_b200.config import EngineConfig, Qwen2Config
    from torchlet_b200.engine import ModelRunner
    from torchlet_b200.engine.loading import build_model

    cfg, w = weights_for(name)
    config = Qwen2Config.from_dict(cfg)
    if schedule is not None:
        config = ScheduledConfig(config, schedule)
    model = build_model(config, {k: v.to(torch.bfloat16) for k, v in w.items()}, dtype)
    page = page_size or tiny_configs.ALL[name][1]["page_size"]
    engine = EngineConfig(dtype=dtype, max_decode_slots=slots, kv_block_size=page, max_num_blocks=num_pages,
                          max_seq_len=max_seq_len or cfg["max_position_embeddings"], max_num_batched_tokens=budget,
                          cuda_graph=cuda_graph)
    return ModelRunner(model, engine)


class ScheduledConfig:
    """A configuration whose model spec runs the layers in another order."""

    def __init__(self, config, schedule):
        self._config, self._schedule = config, schedule

    def __getattr__(self, name):
        return getattr(self._config, name)

    def model_spec(self):
        import dataclasses

        from torchlet_b200.config import ScheduleEntry

        spec = self._config.model_spec()
        return dataclasses.replace(spec, schedule=tuple(ScheduleEntry(l, c) for l, c in self._schedule))


def replay(runner, rid, ids, cuts):
    """Feed ``ids`` of one request in portions of the given sizes, asking for every
    position's logits; returns [len(ids), vocab] on the CPU."""
    from torchlet_b200.engine import StepEntry

    assert sum(cuts) == len(ids)
    runner.admit(rid)
    out, start = [], 0
    for size in cuts:
        logits = runner.step([StepEntry(rid, ids[start:start + size], list(range(size)))])
        out.append(logits.cpu().clone())
        start += size
    runner.finish(rid)
    runner.cache.check()
    return torch.cat(out)


def changing_cuts(length: int, seed: int = 0):
    """Portions of changing size, down to two tokens, that add up to ``length``."""
    pattern = [7, 2, 5, 3, 16, 2, 9, 1, 4, 33, 2, 6]
    cuts, i = [], seed
    while sum(cuts) < length:
        cuts.append(min(pattern[i % len(pattern)], length - sum(cuts)))
        i += 1
    return cuts


def assert_close(got, want, dtype: str, what: str = ""):
    """Row by row (one row = the logits of one position): the largest difference of a row against
    the largest |logit| of THAT row, so that an error confined to one position or one request
    cannot hide under the largest logit of the whole comparison."""
    assert got.shape == want.shape, f"{what}: shapes {tuple(got.shape)} and {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    got, want = got.reshape(-1, got.shape[-1]).double(), want.reshape(-1, want.shape[-1]).double()
    err = (got - want).abs().amax(dim=1)
    scale = want.abs().amax(dim=1)
    ratio = err / scale
    worst = int(ratio.argmax())
    assert ratio[worst] <= TOLERANCE[dtype], (
        f"{what}: row {worst}: max |diff| {err[worst]:.3e} > {TOLERANCE[dtype]:.1e} * {scale[worst]:.3f}")


class KernelCalls:
    """Counts the calls of the kernel wrappers in ``torchlet_b200.ops`` while it is active, so
    that a test can say which kernels its comparison went through."""

    NAMES = ("attention_mma", "attention_tc", "attention_generic", "gemm_tc", "gemm_tc_deferred", "gemm_simt",
             "finish_qkv_rope", "finish_accum_norm")

    def __enter__(self):
        from torchlet_b200 import ops

        self.counts = {name: 0 for name in self.NAMES}
        self.decode_splits = []
        self.prompt_splits = []
        self.side_by_side = 0  # decode attention launched beside the prompt portions' kernel
        self._saved = {name: getattr(ops, name) for name in self.NAMES}
        for name, fn in self._saved.items():
            setattr(ops, name, self._wrap(name, fn))
        return self

    def _wrap(self, name, fn):
        def counted(*args, **kwargs):
            self.counts[name] += 1
            if name == "attention_mma" and kwargs.get("rows16"):
                self.decode_splits.append(kwargs.get("splits", 1))
                self.side_by_side += bool(kwargs.get("late_wait"))
            if name == "attention_tc":
                self.prompt_splits.append(kwargs.get("splits", 1))
            return fn(*args, **kwargs)

        return counted

    def __exit__(self, *exc):
        from torchlet_b200 import ops

        for name, fn in self._saved.items():
            setattr(ops, name, fn)
        return False
