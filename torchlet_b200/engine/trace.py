"""Trace replay: feeds given token ids through the model step by step and writes
logits.  It samples nothing and owns no forward pass, cache or loader: it drives the
same model, step function, cache manager and kernels that generation uses.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``DIR/<step>.f32`` holds the logits at the
wanted places, in the order of the entries and of ``want``, little-endian float32
``[wanted, vocab]``.  After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def parse_args(argv=None):
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--out", required=True, help="folder the logits are written to")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=16,
                        help="tokens per cache page (any size the kernels take)")
    parser.add_argument("--max-live", type=int, default=8, help="most requests live at a time")
    return parser.parse_args(argv)


def main(argv=None, stdin=None, stdout=None) -> int:
    args = parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    if args.page_size <= 0:
        raise SystemExit("--page-size must be positive")
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    import numpy as np

    from .. import ops
    from ..config import EngineConfig
    from .loading import load_model
    from .runner import ModelRunner, StepEntry

    print("[trace_run] loading the model and compiling kernels if needed ...", file=sys.stderr, flush=True)
    model = load_model(args.model, args.dtype)
    max_tokens = -(-max(args.max_tokens, 64) // 64) * 64
    # pages for that many tokens; a page size that does not divide 64 may leave every live request
    # one page short of its rounded count, so those get one page each on top
    num_pages = -(-max_tokens // args.page_size) + (0 if 64 % args.page_size == 0 else args.max_live)
    max_pos = model.spec.max_position_embeddings
    config = EngineConfig(
        dtype=args.dtype,
        max_decode_slots=args.max_live,
        kv_block_size=args.page_size,
        max_num_blocks=num_pages + 1,
        max_seq_len=min(max_tokens, max_pos),
        max_num_batched_tokens=max(2048, min(max_tokens, max_pos)),
        cuda_graph=True,  # steps of single tokens replay the captured decode step, as serving does
    )
    runner = ModelRunner(model, config)
    print("[trace_run] ready", file=sys.stderr, flush=True)

    for line in stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            if not runner.cache.has(item["id"]):
                runner.admit(item["id"])
            entries.append(StepEntry(item["id"], item["tokens"], item.get("want", [])))
        logits = runner.step(entries)
        if logits is not None:
            array = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            ops.raise_on_wait_errors()  # before anything of this step is written
            array.tofile(out_dir / f"{step}.f32")
        for request_id in record.get("end", []):
            if runner.cache.has(request_id):
                runner.finish(request_id)
        print(f"done {step}", file=stdout, flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
