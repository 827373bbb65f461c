"""Two further workloads, run through the engine's own loop (scheduler -> step function):

``interleave14b``  Qwen2.5-14B layer sizes (48 layers, hidden 5120, 40 heads in 8 groups of 5,
    head_dim 128, intermediate 13824, vocabulary 152064, untied; random bfloat16 weights, seed 6):
    eight 4,096-token prompts are read in portions of 512 tokens beside 32 requests that decode.
    Every timed step is a MIXED step: 32 single tokens and one 512-token portion in one batch.
    (The reference has no such forward: it runs whole prompts and decode tokens as two separate
    forwards, v10_triton_paged_gqa/engine.py:105-133.)

``stress05b``  Qwen2.5-0.5B layer sizes (24 layers, hidden 896, 14 heads in 2 groups of 7,
    head_dim 64, intermediate 4864, vocabulary 151936, tied; the reference's own example size,
    v10_triton_paged_gqa/llm.py:113-140; random bfloat16 weights, seed 5): 256 requests, prompt
    lengths uniform in [16, 1024], output lengths uniform in [16, 512], arriving in a seeded
    Poisson order while others run, greedy and temperature 0.7 mixed, in a pool that is too small
    for all live requests at full length.  All must finish and every page and slot must come back;
    in float32 a sample of the requests must give the very tokens it gives when run alone.

    python -m torchlet_b200.benchmarks.workloads interleave14b|stress05b [--layers N] [--requests N]

Both print one JSON object.
"""
from __future__ import annotations

import argparse
import json
import random
import time

import torch

from .common import QWEN25_05B, QWEN25_14B


def _model(cfg: dict, layers: int, seed: int, dtype: str = "bfloat16"):
    from ..config import Qwen2Config
    from ..engine.loading import build_model
    from ..weights import random_tensors

    config = Qwen2Config.from_dict(dict(cfg, num_hidden_layers=layers))
    tensors = random_tensors(config, seed, std=0.02, norm_std=0.0, dtype="bfloat16", device="cuda:0")
    model = build_model(config, tensors, dtype)
    del tensors
    torch.cuda.empty_cache()
    return model


def _sizes(cfg: dict, layers: int):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = H // nh
    layer_matrices = (nh + 2 * nkv) * d * H + H * nh * d + 3 * I * H  # parameters of a layer's products
    return {"layer_matrices": layer_matrices, "head": V * H, "kv_bytes_per_token": 2 * layers * nkv * d * 2,
            "nh": nh, "d": d, "layers": layers}


# ------------------------------------------------------------------ interleave14b
def interleave14b(layers: int = 48, decoders: int = 32, prompts: int = 8, prompt_len: int = 4096, portion: int = 512,
                  decoder_context: int = 2048, peaks: dict | None = None) -> dict:
    """Two token budgets are timed: ``decoders + portion`` (every step holds a full 512-token
    portion beside the 32 decode tokens: 544 rows, which the 128-row tiles of the products cover
    as 640) and ``portion`` (the step's tokens fill whole tiles: 480-token portions beside the
    32 decode tokens)."""
    from ..config import EngineConfig
    from ..engine.engine import Engine
    from ..engine.scheduler import Request
    from ..sampling import SamplingParams

    cfg = QWEN25_14B
    model = _model(cfg, layers, seed=6)
    page, context = 16, 8192
    budgets = {"full_portions": decoders + portion, "whole_tiles": portion}
    decode_steps = sum(prompts * -(-prompt_len // (b - decoders)) for b in budgets.values()) + 64
    tokens_held = decoders * (decoder_context + decode_steps + 64) + prompts * (prompt_len + 64)
    engine = Engine(model, EngineConfig(
        dtype="bfloat16", max_decode_slots=decoders + prompts, kv_block_size=page, max_seq_len=context,
        max_num_blocks=tokens_held // page + decoders + prompts + 1, max_num_batched_tokens=4096))
    generator = torch.Generator().manual_seed(6)
    draw = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=generator).tolist()
    running = [Request(draw(decoder_context), SamplingParams(max_new_tokens=decode_steps, ignore_eos=True))
               for _ in range(decoders)]
    engine.add_requests(running)
    while any(r.num_computed < decoder_context for r in running):  # their prompts, untimed
        engine.step()
    for _ in range(4):  # decode-only steps: warm-up, graph capture
        engine.step()
    sizes = _sizes(cfg, layers)
    stats = engine.scheduler.stats
    record = {"workload": "interleave14b",
              "metric": "mixed step: 32 decode tokens beside a portion of a 4,096-token prompt (Qwen2.5-14B layer sizes)"}
    everyone = list(running)
    for name, budget in budgets.items():
        # the token budget of a step: every decoder's token and ONE portion of a prompt
        engine.scheduler.max_num_batched_tokens = budget
        cut = budget - decoders
        # a prompt is done with its first sampled token, so the decoders stay 32
        fresh = [Request(draw(prompt_len), SamplingParams(max_new_tokens=1, ignore_eos=True)) for _ in range(prompts)]
        everyone += fresh
        engine.add_requests(fresh)
        engine.step()  # the first mixed step is the warm-up of its shapes
        torch.cuda.synchronize()
        times, mixes, contexts = [], [], []
        while any(r.num_computed < prompt_len for r in fresh):
            before = (stats.prefill_tokens, stats.decode_tokens)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            engine.step()
            end.record()
            torch.cuda.synchronize()
            mix = (stats.prefill_tokens - before[0], stats.decode_tokens - before[1])
            if mix == (cut, decoders):
                times.append(begin.elapsed_time(end))
                contexts.append(sum(r.num_tokens for r in running) / decoders)
            mixes.append(mix)
        if not times:
            raise RuntimeError(f"no step held {decoders} decode tokens beside a {cut}-token portion: {mixes[:8]}")
        ms = sorted(times)[len(times) // 2]  # the median step
        # what such a step must read and compute
        decode_context = sum(contexts) / len(contexts)  # the decoders' cached tokens, on average
        portion_context = (prompt_len - cut) / 2  # a portion's cached prefix, on average
        weight_bytes = 2 * (layers * sizes["layer_matrices"] + sizes["head"])
        kv_bytes = sizes["kv_bytes_per_token"] * (decoders * decode_context + portion_context + cut)
        tokens = decoders + cut
        gemm_flops = 2.0 * tokens * layers * sizes["layer_matrices"] + 2.0 * decoders * sizes["head"]
        attention_flops = layers * 4.0 * sizes["nh"] * sizes["d"] * (
            decoders * decode_context + cut * (portion_context + cut / 2))
        flops = gemm_flops + attention_flops
        entry = {"token_budget": budget, "portion": cut, "ms_per_step": round(ms, 3), "timed_steps": len(times),
                 "steps": len(mixes), "decode_tok_s": round(decoders / (ms / 1e3), 1),
                 "prefill_tok_s": round(cut / (ms / 1e3), 1), "tok_s": round(tokens / (ms / 1e3), 1),
                 "decoder_context": int(decode_context), "bytes_per_step": int(weight_bytes + kv_bytes),
                 "flops_per_step": flops, "achieved_gbs": round((weight_bytes + kv_bytes) / (ms / 1e3) / 1e9, 1),
                 "achieved_tflops": round(flops / (ms / 1e3) / 1e12, 1)}
        if peaks:
            entry["hbm_frac"] = round(entry["achieved_gbs"] / peaks["hbm_gbs"], 4)
            entry["tensor_frac"] = round(entry["achieved_tflops"] / peaks["bf16_tflops"], 4)
            # the step can be no faster than the slower of its two bounds
            bound_ms = max((weight_bytes + kv_bytes) / peaks["hbm_gbs"] / 1e6, flops / peaks["bf16_tflops"] / 1e9)
            entry["roofline_frac"] = round(bound_ms / ms, 4)
        record[name] = entry
    record["tok_s"] = record["full_portions"]["tok_s"]
    record["config"] = {"model": "Qwen2.5-14B layer sizes, random weights seed 6", "layers": layers,
                        "layers_of_configuration": cfg["num_hidden_layers"], "hidden_size": cfg["hidden_size"],
                        "intermediate_size": cfg["intermediate_size"], "num_attention_heads": cfg["num_attention_heads"],
                        "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": sizes["d"],
                        "vocab_size": cfg["vocab_size"], "context": context, "kv_page_size": page, "decoders": decoders,
                        "prompts": prompts, "prompt_len": prompt_len, "portion": portion, "dtype": "bf16",
                        "data": "synthetic"}
    engine.scheduler.max_num_batched_tokens = 4096
    engine.run()  # let everything finish; every page and slot must come back
    engine.runner.cache.check()
    record["all_finished"] = all(r.error is None for r in everyone) and not engine.runner.cache.live_requests()
    return record


# ---------------------------------------------------------------------- stress05b
def _stress_requests(count: int, seed: int, vocab: int):
    from ..engine.scheduler import Request
    from ..sampling import SamplingParams

    rng = random.Random(seed)
    requests, arrivals, now = [], [], 0.0
    for i in range(count):
        prompt = [rng.randrange(vocab) for _ in range(rng.randint(16, 1024))]
        params = SamplingParams(max_new_tokens=rng.randint(16, 512), temperature=rng.choice([0.0, 0.7]), seed=9000 + i,
                                ignore_eos=True)
        requests.append(Request(prompt, params))
        now += rng.expovariate(1.0)  # a Poisson process: one arrival a step on average
        arrivals.append(now)
    return requests, arrivals


def _warm_up(engine, slots: int, vocab: int) -> None:
    """Untimed: as many short requests as there are slots, of different lengths, so that the decode
    step is captured for every batch-size bucket from the full batch down to one request; the
    counters start again afterwards."""
    from ..engine.scheduler import Request, SchedulerStats
    from ..sampling import SamplingParams

    rng = random.Random(99)
    engine.generate([Request([rng.randrange(vocab) for _ in range(8)],
                             SamplingParams(max_new_tokens=3 + i % 24, ignore_eos=True)) for i in range(slots)])
    engine.scheduler.stats = SchedulerStats()
    engine.runner.graph_steps = 0
    engine.steps_ahead = 0
    for pool in engine.runner.cache.pools:
        pool.peak_held = 0


def _run_stress(engine, requests, arrivals) -> dict:
    """Runs the engine's loop while requests arrive at their times.  The unit of time is one
    scheduling decision of the loop; when nothing is left to do the next request arrives at once."""
    pending = list(zip(arrivals, requests))
    clock = [0]

    def poll():
        if not pending:
            return None
        arrived = []
        while pending and (pending[0][0] <= clock[0] or not (arrived or engine.scheduler.has_work())):
            arrived.append(pending.pop(0)[1])
        clock[0] += 1
        return arrived

    torch.cuda.synchronize()
    start = time.perf_counter()
    engine.run(poll)
    torch.cuda.synchronize()
    return {"seconds": time.perf_counter() - start, "steps": engine.scheduler.stats.steps}


def stress05b(layers: int = 24, count: int = 256, sample: int = 6, check_float32: bool = True) -> dict:
    from ..config import EngineConfig
    from ..engine.engine import Engine

    cfg = QWEN25_05B
    slots, page, context = 48, 16, 1536
    # room for about two thirds of the slots at their mean length: pages do run out
    num_blocks = int(slots * 0.66 * (520 + 264) / page) + 1
    record = {"workload": "stress05b", "metric": "output tok/s under continuous batching (256 requests arriving)"}
    outputs = {}
    for dtype in ("bfloat16", "float32") if check_float32 else ("bfloat16",):
        model = _model(cfg, layers, seed=5, dtype=dtype)
        engine = Engine(model, EngineConfig(dtype=dtype, max_decode_slots=slots, kv_block_size=page, max_seq_len=context,
                                            max_num_blocks=num_blocks, max_num_batched_tokens=2048))
        requests, arrivals = _stress_requests(count, seed=5, vocab=cfg["vocab_size"])
        _warm_up(engine, slots, cfg["vocab_size"])
        run = _run_stress(engine, requests, arrivals)
        stats = engine.scheduler.stats
        engine.runner.cache.check()
        produced = sum(len(r.output_tokens) for r in requests)
        ok = (all(r.error is None and len(r.output_tokens) == r.params.max_new_tokens for r in requests)
              and not engine.runner.cache.live_requests()
              and engine.runner.cache.pools[0].num_free == num_blocks - 1 and engine.runner.cache.num_free_slots == slots)
        outputs[dtype] = [list(r.output_tokens) for r in requests]
        entry = {"all_finished_and_everything_returned": ok, "seconds": round(run["seconds"], 3), "steps": run["steps"],
                 "output_tokens": produced, "prompt_tokens": sum(len(r.prompt_tokens) for r in requests),
                 "output_tok_s": round(produced / run["seconds"], 1),
                 "total_tok_s": round((stats.prefill_tokens + stats.decode_tokens) / run["seconds"], 1),
                 "preemptions": stats.preemptions, "recomputed_tokens": stats.prefill_tokens - sum(
                     len(r.prompt_tokens) for r in requests),
                 "peak_running": stats.peak_running, "peak_pages": stats.peak_pages,
                 "graph_steps": engine.runner.graph_steps}
        if dtype == "float32":  # a sample of the requests, each run alone: the very same tokens
            alone = Engine(model, EngineConfig(dtype=dtype, max_decode_slots=1, kv_block_size=page, max_seq_len=context,
                                               max_num_batched_tokens=2048, cuda_graph=False))
            again, _ = _stress_requests(count, seed=5, vocab=cfg["vocab_size"])
            picks = random.Random(7).sample(range(count), min(sample, count))
            same = 0
            for i in picks:
                alone.generate([again[i]])
                same += again[i].output_tokens == outputs[dtype][i]
            entry["alone_equal"] = f"{same} of {len(picks)}"
            entry["all_finished_and_everything_returned"] = ok and same == len(picks)
            del alone
        record[dtype] = entry
        del engine, model
        torch.cuda.empty_cache()
    record["value"] = record["bfloat16"]["output_tok_s"]
    record["unit"] = "tok/s"
    record["config"] = {"model": "Qwen2.5-0.5B layer sizes, random weights seed 5", "layers": layers,
                        "layers_of_configuration": cfg["num_hidden_layers"], "hidden_size": cfg["hidden_size"],
                        "intermediate_size": cfg["intermediate_size"], "num_attention_heads": 14,
                        "num_key_value_heads": 2, "head_dim": 64, "vocab_size": cfg["vocab_size"], "tied": True,
                        "requests": count, "prompt_len": "uniform 16..1024", "output_len": "uniform 16..512",
                        "arrivals": "Poisson, one a step on average, seed 5", "sampling": "greedy and temperature 0.7",
                        "max_decode_slots": slots, "kv_page_size": page, "pool_pages": num_blocks, "data": "synthetic"}
    return record


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("workload", choices=["interleave14b", "stress05b"])
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    parser.add_argument("--requests", type=int, default=256, help="stress05b: number of requests")
    parser.add_argument("--no-float32", action="store_true", help="stress05b: leave out the float32 run and its check")
    args = parser.parse_args(argv)
    if args.workload == "interleave14b":
        record = interleave14b(layers=args.layers or 48)
    else:
        record = stress05b(layers=args.layers or 24, count=args.requests, check_float32=not args.no_float32)
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
