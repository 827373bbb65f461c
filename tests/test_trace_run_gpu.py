"""bin/trace_run as a user runs it: a model folder, steps on standard input, logits files
out; compared with the plain implementation for both dtypes."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import harness
import tiny_configs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run(tmp_path, dtype):
    cfg, w = harness.weights_for("B")
    folder = tiny_configs.write_model_dir(tmp_path / "model", cfg, {k: v.to(torch.bfloat16) for k, v in w.items()})
    a, want_a = harness.plain_logits("B", 70, 31)
    b, want_b = harness.plain_logits("B", 45, 32)
    c, want_c = harness.plain_logits("B", 64, 33)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [0, 49]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[50:52], "want": [1]}, {"id": "b", "tokens": b[:45], "want": list(range(45))}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[52:53]}], "end": []},  # nothing wanted: no file
        {"step": 3, "entries": [{"id": "c", "tokens": c[:64], "want": [63]}, {"id": "a", "tokens": a[53:70], "want": [16]}], "end": ["a", "c"]},
    ]
    out = tmp_path / "out"
    proc = subprocess.run(
        [str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "192"],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(4)]
    vocab = cfg["vocab_size"]
    read = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab))
    assert not (out / "2.f32").exists()
    harness.assert_close(read(0), want_a[[0, 49]], dtype, "step 0")
    harness.assert_close(read(1), torch.cat([want_a[[51]], want_b]), dtype, "step 1")
    harness.assert_close(read(3), torch.cat([want_c[[63]], want_a[[69]]]), dtype, "step 3")


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("B", "bfloat16"), ("E", "bfloat16")])
def test_trace_run_single_token_steps_beside_portions_with_pages_used_again(tmp_path, name, dtype):
    """A longer trace through the program itself: the last 32 tokens of a request one by one
    (steps of single tokens replay the captured decode step, as serving does), single tokens of one
    request beside portions of another (a mixed step), two requests decoding together, and a pool
    so small that the third request gets the pages the first gave back."""
    cfg, w = harness.weights_for(name)
    folder = tiny_configs.write_model_dir(tmp_path / "model", cfg, {k: v.to(torch.bfloat16) for k, v in w.items()})
    page = tiny_configs.ALL[name][1]["page_size"]
    x, want_x = harness.plain_logits(name, 120, 41)
    y, want_y = harness.plain_logits(name, 100, 42)
    z, want_z = harness.plain_logits(name, 90, 43)
    steps, expect = [], []

    def add(entries, end=()):
        steps.append({"step": len(steps), "entries": [{"id": i, "tokens": t, "want": wt} for i, t, wt, _ in entries],
                      "end": list(end)})
        rows = [want[[first + k for k in wt]] for _, _, wt, (want, first) in entries if wt]
        expect.append(torch.cat(rows) if rows else None)

    add([("x", x[:88], [0, 87], (want_x, 0))])
    fed_y = 0
    for k in range(88, 120):  # the last 32 tokens of x one by one; from the 10th on beside portions of y
        entries = [("x", x[k:k + 1], [0], (want_x, k))]
        if k >= 98 and fed_y < 100:
            size = [7, 2, 11, 5][k % 4]
            size = min(size, 100 - fed_y - 20)
            if size > 0:
                entries.append(("y", y[fed_y:fed_y + size], list(range(size)), (want_y, fed_y)))
                fed_y += size
        add(entries, end=["x"] if k == 119 else [])
    add([("z", z[:60], [59], (want_z, 0))])  # x is gone: z takes pages x gave back
    fed_z = 60
    while fed_y < 100 or fed_z < 90:  # y and z decode together, one token each
        entries, end = [], []
        if fed_y < 100:
            entries.append(("y", y[fed_y:fed_y + 1], [0], (want_y, fed_y)))
            fed_y += 1
            end += ["y"] if fed_y == 100 else []
        if fed_z < 90:
            entries.append(("z", z[fed_z:fed_z + 1], [0], (want_z, fed_z)))
            fed_z += 1
            end += ["z"] if fed_z == 90 else []
        add(entries, end)
    out = tmp_path / "out"
    # x (120 -> 128) and y (100 -> 128) live together, then y and z (90 -> 128): 256 tokens at most
    proc = subprocess.run(
        [str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "256",
         "--page-size", str(page), "--max-live", "4"],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.count("done ") == len(steps)
    vocab = cfg["vocab_size"]
    for i, want in enumerate(expect):
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab))
        harness.assert_close(got, want, dtype, f"{name} step {i}")
