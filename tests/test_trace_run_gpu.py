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
