#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens a second at Qwen2.5-7B layer sizes
with random bfloat16 weights (batch 8, context 4096 by default), with the prefill of a
2,048-token prompt, decode at batch 1 and 64, the roofline fractions and the clocks seen.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  ``value`` times
the step function on the device with CUDA events (host -> device copy of the step's
metadata included); ``e2e`` times the same decode steps through the Python entry point
(``LLM`` -> engine -> scheduler), host tokens in and out, by the wall clock.  Inputs are
seeded synthetic token ids; the cached context of the decode runs is seeded random keys
and values.  Every step reads all weights (15 GB), far more than the 126 MB L2, so no
L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-7B layer sizes (the reference arm reads them here, so that it imports nothing of this package)
QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 152064, "hidden_size": 3584, "intermediate_size": 18944,
    "num_hidden_layers": 28, "num_attention_heads": 28, "num_key_value_heads": 4, "max_position_embeddings": 32768,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": False,
}


FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks, source = dict(FALLBACK_PEAKS), "fallback"
    try:
        with open(path) as handle:
            raw = json.load(handle)
        for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if isinstance(raw.get(key), (int, float)) and raw[key] > 0:
                peaks[key] = float(raw[key])
                source = "measured"
    except (OSError, ValueError):
        pass
    return peaks, source


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons.  It is started before the warm-up (the
    tool needs a moment to come up) and told when the timed region begins and ends; the record
    is made of the samples that fall inside the region, or, if the region was shorter than three
    sampling periods, of the samples since the warm-up began (the GPU was under the same load)."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    PERIOD_MS = 20

    def __init__(self):
        self.proc = None
        self.begin = self.end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms",
                 str(self.PERIOD_MS)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark_begin(self):
        self.begin = time.time()

    def mark_end(self):
        self.end = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        if self.end is None:
            self.mark_end()
        time.sleep(2 * self.PERIOD_MS / 1e3)  # let the last sample of the region be written
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime

        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        samples = []  # (seconds since the epoch or None, clock, reasons)
        max_clock = None
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clock, max_clock = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            try:
                when = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
            except ValueError:
                when = None
            samples.append((when, clock, {n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")}))
        inside = [x for x in samples if x[0] is not None and self.begin is not None and self.begin <= x[0] <= self.end]
        used, span = (inside, "timed region") if len(inside) >= 3 else (samples, "warm-up and timed region")
        clocks = sorted(x[1] for x in used)
        reasons = set().union(*[x[2] for x in used]) if used else set()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks), "samples_in_timed_region": len(inside),
                "span": span, "period_ms": self.PERIOD_MS}


def config_record(cfg: dict, layers: int, batch: int, context: int) -> dict:
    """The ``config`` of the JSON line; both arms print the same keys."""
    return {
        "model": "Qwen2.5-7B layer sizes, random weights seed 4", "global_batch": batch, "seq_len": context,
        "parallelism": "single GPU", "layers": layers, "layers_of_configuration": cfg["num_hidden_layers"],
        "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
        "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
        "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "vocab_size": cfg["vocab_size"],
        "kv_page_size": 16, "prefill_tokens": 2048, "cuda_graph": True,
        "l2": "each step reads 15 GB of weights, larger than L2; no flush",
        "context": "cached keys/values are seeded random numbers (ours); prompts of seeded random ids (reference)",
    }


def model_numbers(cfg: dict, layers: int):
    """Parameters a decode step reads, KV bytes per token, and flops of a prefill."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = H // nh
    per_layer = (nh + 2 * nkv) * d * H + (nh + 2 * nkv) * d + H * nh * d + 3 * I * H + 2 * H
    read_params = layers * per_layer + V * H + H  # layers + LM head + final norm
    kv_bytes_per_token = 2 * layers * nkv * d * 2

    def prefill_flops(tokens: int) -> float:
        gemm = 2.0 * tokens * layers * ((nh + 2 * nkv) * d * H + H * nh * d + 3 * I * H)
        attention = layers * 4.0 * nh * d * tokens * (tokens + 1) / 2  # causal q.k and p.v
        head = 2.0 * V * H  # one row of logits
        return gemm + attention + head

    return read_params, kv_bytes_per_token, prefill_flops


def time_decode(model, batch: int, context: int, steps: int, warmup: int, clock=None):
    """Device time of ``steps`` decode steps of ``batch`` requests ending at ``context``."""
    import torch

    from torchlet_b200 import ops
    from torchlet_b200.benchmarks import common
    from torchlet_b200.config import EngineConfig
    from torchlet_b200.engine import ModelRunner, StepEntry
    from torchlet_b200.sampling import SampleSpec

    page = 16
    start_len = context - steps - warmup
    config = EngineConfig(dtype="bfloat16", max_decode_slots=batch, kv_block_size=page, max_seq_len=context,
                          max_num_blocks=batch * (-(-context // page)) + 1, max_num_batched_tokens=2048)
    runner = ModelRunner(model, config)
    ids = [f"d{i}" for i in range(batch)]
    common.fill_context(runner, ids, start_len, seed=17)
    vocab = model.spec.vocab_size
    generator = torch.Generator().manual_seed(batch)
    tokens = torch.randint(0, vocab, (steps + warmup, batch), generator=generator).tolist()

    def step(k):
        entries = [StepEntry(rid, [tokens[k][i]], sample=SampleSpec(0.0, i, k)) for i, rid in enumerate(ids)]
        return runner.run(entries)

    if clock:
        clock.start()
    for k in range(warmup):
        step(k)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = ops.launch_count
    if clock:
        clock.mark_begin()
    begin.record()
    for k in range(warmup, warmup + steps):
        step(k)
    end.record()
    torch.cuda.synchronize()
    if clock:
        clock.mark_end()
    stats = clock.stop() if clock else None
    ms = begin.elapsed_time(end)
    launches = ops.launch_count - launches
    h2d_bytes = runner.h2d_bytes_last_step  # the command block of a steady decode step
    mean_context = start_len + warmup + steps / 2
    for rid in ids:
        runner.finish(rid)
    del runner
    torch.cuda.empty_cache()
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "h2d_bytes": h2d_bytes, "mean_context": mean_context, "clocks": stats}


def time_prefill(model, tokens: int, repeats: int):
    import torch

    from torchlet_b200.config import EngineConfig
    from torchlet_b200.engine import ModelRunner, StepEntry
    from torchlet_b200.sampling import SampleSpec

    config = EngineConfig(dtype="bfloat16", max_decode_slots=2, kv_block_size=16, max_seq_len=tokens + 16,
                          max_num_batched_tokens=tokens)
    runner = ModelRunner(model, config)
    generator = torch.Generator().manual_seed(3)
    best = None
    for r in range(repeats + 2):
        prompt = torch.randint(0, model.spec.vocab_size, (tokens,), generator=generator).tolist()
        runner.admit("p")
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        result = runner.run([StepEntry("p", prompt, sample=SampleSpec())])
        end.record()
        torch.cuda.synchronize()
        result.tokens.tolist()
        runner.finish("p")
        ms = begin.elapsed_time(end)
        if r >= 2:
            best = ms if best is None else min(best, ms)
    del runner
    torch.cuda.empty_cache()
    return best


def time_e2e(model, batch: int, context: int, steps: int, warmup: int):
    """The same decode steps through the Python entry point: ``LLM`` -> engine -> scheduler
    -> step function, host token ids in, host token ids out, by the wall clock."""
    import torch

    from torchlet_b200 import LLM, SamplingParams
    from torchlet_b200.engine.scheduler import Request

    page = 16
    llm = LLM.from_model(model, max_decode_slots=batch, kv_block_size=page, max_seq_len=context,
                         max_num_blocks=batch * (-(-context // page)) + 1, max_num_batched_tokens=2048)
    engine = llm.engine
    # requests that finish their prompt early decode while the others still read theirs:
    # leave room so that none reaches its last token inside the timed steps
    slack = 2 * (batch * context // 2048 + 2)
    prompt_len = context - steps - warmup - slack - 1
    generator = torch.Generator().manual_seed(5)
    params = SamplingParams(max_new_tokens=steps + warmup + slack + 1, ignore_eos=True)
    requests = [Request(torch.randint(0, model.spec.vocab_size, (prompt_len,), generator=generator).tolist(),
                        SamplingParams(**vars(params))) for _ in range(batch)]
    engine.add_requests(requests)
    while any(r.num_computed < prompt_len for r in requests):  # prompts, in portions (untimed)
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    graph_before = engine.runner.graph_steps
    produced = sum(len(r.output_tokens) for r in requests)
    # every request gets exactly ``steps`` more tokens, so the timed call is ``steps`` full decode steps
    for r in requests:
        r.params.max_new_tokens = len(r.output_tokens) + steps
    import gc

    gc.collect()
    gc.disable()  # a collection inside a timed region of a few dozen milliseconds would be most of it
    try:
        start = time.perf_counter()
        engine.run()  # the loop behind LLM.generate: schedule, step, tokens back to the host, until all are done
        torch.cuda.synchronize()
        seconds = time.perf_counter() - start
    finally:
        gc.enable()
    produced = sum(len(r.output_tokens) for r in requests) - produced
    graph_steps = engine.runner.graph_steps - graph_before
    if produced != batch * steps:
        raise RuntimeError(f"e2e run produced {produced} tokens, expected {batch * steps}")
    h2d_bytes = engine.runner.h2d_bytes_last_step  # the command block of a steady decode step
    ahead = engine.steps_ahead
    del llm, engine
    torch.cuda.empty_cache()
    return {"tok_s": produced / seconds, "ms_per_step": seconds * 1e3 / steps, "h2d_bytes": h2d_bytes,
            "d2h_bytes": batch * 4, "graph_steps": graph_steps, "steps_launched_ahead": ahead}


def _write_reference_folder(folder: str, cfg: dict, layers: int, context: int, seed: int) -> None:
    """A model folder the reference can load: config.json, random weights (the same
    generator and seed as our arm), and a word-level tokenizer whose word ``t<i>`` is token i
    and whose chat template is the message text itself, so a prompt's length is exact."""
    import torch
    from safetensors.torch import save_file
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from torchlet_b200.config import Qwen2Config
    from torchlet_b200.weights import random_tensors

    os.makedirs(folder, exist_ok=True)
    raw = dict(cfg, num_hidden_layers=layers, max_position_embeddings=context)
    config = Qwen2Config.from_dict(raw)
    tensors = random_tensors(config, seed, std=0.02, norm_std=0.0, dtype="bfloat16", device="cuda:0")
    save_file({k: v.cpu().contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    del tensors
    torch.cuda.empty_cache()
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(dict(raw, torch_dtype="bfloat16"), handle)
    words = 4096  # prompts use only the first ids
    vocab = {f"t{i}": i for i in range(words)}
    vocab["<|im_end|>"] = words
    vocab["<unk>"] = words + 1
    tokenizer = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tokenizer.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    PreTrainedTokenizerFast(tokenizer_object=tokenizer, eos_token="<|im_end|>", unk_token="<unk>",
                            chat_template="{% for m in messages %}{{ m['content'] }}{% endfor %}").save_pretrained(folder)


def reference_arm(args) -> int:
    """The UNMODIFIED reference (installed under baseline/_ref) through its own public API:
    ``LLM(model_id, max_decode_slots=batch).generate(list[str], max_new_tokens)``
    (v10_triton_paged_gqa/llm.py:20-110).  The only thing supplied from outside is the
    package ``modelscope``, which is not installed here and would download the model from
    the network (llm.py:9, 34): a stand-in module whose ``snapshot_download`` returns a
    local folder with random weights of the same configuration and seed.  Decode tokens a
    second are taken from two ``generate`` calls that differ only in ``max_new_tokens``
    (same prompts, same prefill), so the prefill cancels out."""
    import asyncio
    import shutil
    import tempfile
    import types

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "torchlet")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/torchlet is not installed"}))
        return 0
    sys.path.insert(0, ref_dir)
    stand_in = types.ModuleType("modelscope")
    stand_in.snapshot_download = lambda model_id, *a, **k: model_id
    sys.modules.setdefault("modelscope", stand_in)
    try:
        import torch
        from torchlet.v10_triton_paged_gqa.llm import LLM
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"impl": "reference",
                          "unavailable": f"the reference's LLM cannot be imported: {type(exc).__name__}: {exc}"}))
        return 0
    cfg = QWEN25_7B
    layers = args.layers or cfg["num_hidden_layers"]
    batch, context, steps = args.batch, args.context, args.steps
    folder = tempfile.mkdtemp(prefix="torchlet_ref_model_")
    try:
        _write_reference_folder(folder, cfg, layers, context, seed=4)
        llm = LLM(folder, max_decode_slots=batch, kv_block_size=16)
        generator = torch.Generator().manual_seed(5)
        short, long = 8, 8 + steps
        prompt_len = context - long - 1
        prompts = [" ".join(f"t{int(i)}" for i in torch.randint(0, 4096, (prompt_len,), generator=generator))
                   for _ in range(batch)]

        async def run(max_new_tokens):
            torch.cuda.synchronize()
            begin = time.perf_counter()
            outputs = await llm.generate(prompts, max_new_tokens=max_new_tokens)
            torch.cuda.synchronize()
            return time.perf_counter() - begin, outputs

        async def everything():
            try:
                await run(4)  # warm-up: Triton compilation, CUDA-graph capture
                clock = ClockSampler()
                clock.start()
                t_short, _ = await run(short)
                t_long, outputs = await run(long)
                stats = clock.stop()
                one = [" ".join(f"t{int(i)}" for i in torch.randint(0, 4096, (2048,), generator=generator))]
                old_prompts = list(prompts)
                prompts[:] = one
                await run(1)  # warm-up of this shape (the reference's Triton kernels autotune per shape)
                t_prefill, _ = await run(1)
                prompts[:] = old_prompts
                return t_short, t_long, t_prefill, stats, outputs
            finally:
                await llm.engine.shutdown()

        t_short, t_long, t_prefill, stats, outputs = asyncio.run(everything())
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"the reference failed to run here: "
                          f"{type(exc).__name__}: {str(exc)[:300]}"}))
        return 0
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    seconds = t_long - t_short
    tok_s = batch * steps / seconds
    print(json.dumps({
        "impl": "reference", "metric": f"decode tok/s @ batch {batch} (Qwen2.5-7B layer sizes, bf16)",
        "value": round(tok_s, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(seconds * 1e3 / steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_record(cfg, layers, batch, context),
        "notes": {"how": "difference of two generate() calls with the same prompts",
                  "modelscope": "stand-in module returning a local folder (no network)"},
        "e2e": {"value": round(tok_s, 1), "unit": "tok/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
        "prefill": {"value": round(2048 / t_prefill, 1), "tokens": 2048, "ms": round(t_prefill * 1e3, 2),
                    "note": "one generate() call of 1 new token, tokenizer included"},
        "clocks": stats, "gpu_launches": None,
    }))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    parser.add_argument("--skip-points", action="store_true", help="leave out prefill, batch 1/64 and e2e")
    parser.add_argument("--workload", choices=["interleave14b", "stress05b"], default=None,
                        help="instead of the headline line: the mixed step at Qwen2.5-14B layer sizes, or 256 requests "
                             "arriving at Qwen2.5-0.5B layer sizes (torchlet_b200/benchmarks/workloads.py)")
    args = parser.parse_args()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU only; --gpus must be 1")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload:
        from torchlet_b200.benchmarks import workloads

        peaks, peak_source = load_peaks()
        if args.workload == "interleave14b":
            record = workloads.interleave14b(layers=args.layers or 48, peaks=peaks)
            record.update(value=record["tok_s"], unit="tok/s")
        else:
            record = workloads.stress05b(layers=args.layers or 24)
        record.update(n_gpus=1, higher_is_better=True, dtype="bf16", data="synthetic", impl="ours",
                      peak_source=peak_source, peaks={k: peaks[k] for k in ("hbm_gbs", "bf16_tflops")})
        print(json.dumps(record))
        return 0
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from torchlet_b200 import ops
    from torchlet_b200.benchmarks import common

    cfg = QWEN25_7B
    layers = args.layers or cfg["num_hidden_layers"]
    peaks, peak_source = load_peaks()
    read_params, kv_per_token, prefill_flops = model_numbers(cfg, layers)
    model = common.build_model(cfg, layers, seed=4)

    clock = ClockSampler()
    main_run = time_decode(model, args.batch, args.context, args.steps, args.warmup, clock)
    wait_error = ops.gemm_tc_error()
    weight_bytes = read_params * 2
    step_bytes = weight_bytes + kv_per_token * main_run["mean_context"] * args.batch
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    record = {
        "metric": "decode tok/s @ batch 8 (Qwen2.5-7B layer sizes, bf16)" if args.batch == 8
        else f"decode tok/s @ batch {args.batch} (Qwen2.5-7B layer sizes, bf16)",
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": config_record(cfg, layers, args.batch, args.context),
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peak_source,
                     "bytes_per_step": int(step_bytes)},
    }
    if wait_error:
        record["kernel_wait_error"] = wait_error
    if not args.skip_points:
        prefill_ms = time_prefill(model, 2048, repeats=3)
        flops = prefill_flops(2048)
        record["prefill"] = {"value": round(2048 / (prefill_ms / 1e3), 1), "tokens": 2048, "ms": round(prefill_ms, 3),
                             "frac": round(flops / (prefill_ms / 1e3) / 1e12 / peaks["bf16_tflops"], 4),
                             "tflops": round(flops / (prefill_ms / 1e3) / 1e12, 1), "peak_tflops": peaks["bf16_tflops"]}
        if peaks.get("bf16_tflops_sustained"):  # the same against the seconds-long cuBLAS figure under the power cap
            record["prefill"]["frac_of_sustained"] = round(
                flops / (prefill_ms / 1e3) / 1e12 / peaks["bf16_tflops_sustained"], 4)
        points = {"note": "each point is the faster of two runs (the host shares its cores with other jobs)"}

        def time_decode_twice(*a):
            return min((time_decode(*a) for _ in range(2)), key=lambda run: run["ms_per_step"])

        for batch in (1, 64):
            run = time_decode_twice(model, batch, args.context, min(args.steps, 64), args.warmup)
            points[f"decode_b{batch}"] = round(run["tok_s"], 1)
            bytes_b = weight_bytes + kv_per_token * run["mean_context"] * batch
            points[f"decode_b{batch}_hbm_frac"] = round(bytes_b / (run["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        # further sizes: decode at other contexts, prefill of other lengths (tok/s and fraction of the peak)
        for context in (1024, 16384):
            for batch in (1, 8, 64):
                run = time_decode_twice(model, batch, context, min(args.steps, 32), args.warmup)
                bytes_b = weight_bytes + kv_per_token * run["mean_context"] * batch
                points[f"decode_b{batch}_ctx{context}"] = round(run["tok_s"], 1)
                points[f"decode_b{batch}_ctx{context}_hbm_frac"] = round(
                    bytes_b / (run["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        for tokens in (512, 8192):
            ms = time_prefill(model, tokens, repeats=2)
            points[f"prefill_{tokens}"] = round(tokens / (ms / 1e3), 1)
            points[f"prefill_{tokens}_frac"] = round(prefill_flops(tokens) / (ms / 1e3) / 1e12 / peaks["bf16_tflops"], 4)
        record["points"] = points
        e2e = time_e2e(model, args.batch, args.context, args.steps, args.warmup)
        record["e2e"] = {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d_bytes"],
                         "d2h_bytes_per_step": e2e["d2h_bytes"], "ms_per_step": round(e2e["ms_per_step"], 4),
                         "graph_steps": e2e["graph_steps"], "steps_launched_ahead": e2e["steps_launched_ahead"]}
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
