"""What each kernel class costs inside the running decode step.

    python -m torchlet_b200.benchmarks.step [--model 7b|14b|0.5b] [--batch 8] [--context 4096] [--steps 64]
                                            [--layers N] [--max-seq-len N] [--only-full]

Builds a model of Qwen2.5-7B (14B, 0.5B) layer sizes with random bfloat16 weights, gives ``batch``
requests a cached context of random keys and values, and times the decode step (CUDA events
around replays of its CUDA graph) once as it is and once with each kernel class replaced by
nothing.  The difference is that class's cost in place, overlap with its neighbours included.
The steps with something left out compute garbage; only their time is used.
"""
from __future__ import annotations

import argparse

import torch

from .. import ops
from ..config import EngineConfig
from ..engine import ModelRunner, StepEntry
from ..sampling import SampleSpec
from .common import SIZES, build_model, fill_context

CLASSES = ("attention_mma", "finish_accum_norm", "finish_qkv_rope")


def time_step(model, batch: int, context: int, steps: int, warmup: int = 4, max_seq_len=None) -> float:
    """Microseconds of one decode step of ``batch`` requests near ``context`` cached tokens.
    ``max_seq_len``: the engine's length limit (default: the context), which the captured decode
    graph is planned for."""
    page = 16
    config = EngineConfig(dtype="bfloat16", max_decode_slots=batch, kv_block_size=page,
                          max_seq_len=max_seq_len or context,
                          max_num_blocks=batch * (-(-context // page)) + 1, max_num_batched_tokens=2048)
    runner = ModelRunner(model, config)
    ids = [f"d{i}" for i in range(batch)]
    fill_context(runner, ids, context - steps - warmup, seed=17)
    tokens = torch.randint(0, model.spec.vocab_size, (steps + warmup, batch)).tolist()

    def step(k):
        runner.run([StepEntry(rid, [tokens[k][i]], sample=SampleSpec(0.0, i, k)) for i, rid in enumerate(ids)])

    for k in range(warmup):
        step(k)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for k in range(warmup, warmup + steps):
        step(k)
    end.record()
    torch.cuda.synchronize()
    for rid in ids:
        runner.finish(rid)
    del runner
    torch.cuda.empty_cache()
    return begin.elapsed_time(end) / steps * 1e3


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--model", choices=sorted(SIZES), default="7b", help="whose layer sizes")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    parser.add_argument("--max-seq-len", type=int, default=None,
                        help="the engine's length limit, if it is to differ from the context")
    parser.add_argument("--only-full", action="store_true", help="time the step as it is and stop")
    args = parser.parse_args(argv)
    cfg, seed = SIZES[args.model]
    args.layers = args.layers or cfg["num_hidden_layers"]
    model = build_model(cfg, args.layers, seed=seed)
    full = time_step(model, args.batch, args.context, args.steps, max_seq_len=args.max_seq_len)
    print(f"Qwen2.5-{args.model} layer sizes, batch {args.batch}, context {args.context}, {args.layers} layers, "
          f"length limit {args.max_seq_len or args.context}")
    print(f"{'full step':32s} {full:9.1f} us")
    for name in () if args.only_full else CLASSES:
        original = getattr(ops, name)
        setattr(ops, name, lambda *a, **k: None)
        try:
            without = time_step(model, args.batch, args.context, args.steps, max_seq_len=args.max_seq_len)
        finally:
            setattr(ops, name, original)
        print(f"{'without ' + name:32s} {without:9.1f} us   {name} costs {full - without:7.1f} us a step, "
              f"{(full - without) / args.layers:6.2f} us a layer")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
