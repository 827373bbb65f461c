"""The debug build (``TORCHLET_B200_DEBUG=1``): kernels compiled with index checks that record the
first bad index and SKIP the access, so nothing faults.  It stands in for a memory checker.  Run
in child processes, because the build variant is chosen when the package is imported:

* the engine's own parity tests pass under it (the two tiny configurations, and the ones that
  run the tensor-core kernels, a window among them; seeded random schedules), with no check
  failing (page ids, positions, slots and token ids stay inside their ranges);
* a kernel handed a page id outside the pool, a position beyond its table, a token id outside
  the vocabulary or a slot outside the range reports it, skips the access, and the process goes on.
  (The bad ids still lie inside the tensors' memory, so that even a missing check could not fault.)
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(code_or_args, timeout=900):
    env = dict(os.environ, TORCHLET_B200_DEBUG="1", PYTHONPATH=os.pathsep.join([ROOT, os.path.join(ROOT, "tests")]))
    return subprocess.run([sys.executable, *code_or_args], cwd=ROOT, env=env, capture_output=True, text=True,
                          timeout=timeout)


def test_parity_tests_pass_in_the_debug_build_and_no_check_fails():
    # (tests/conftest.py asserts after every test of a debug build that no check has fired)
    proc = _run(["-m", "pytest", "-q", "-x", "-m", "gpu", "tests/test_replay_gpu.py", "tests/test_slot_records_gpu.py",
                 "tests/test_random_schedules_gpu.py", "-k",
                 "A-float32 or B-bfloat16 or B-float32 or D-bfloat16 or F-bfloat16 or E-bfloat16", "-p", "no:cacheprovider"])
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    assert "passed" in proc.stdout and "failed" not in proc.stdout


CHECKS = r'''
import torch
from torchlet_b200 import ops
from torchlet_b200.csrc.build import DEBUG_BUILD
assert DEBUG_BUILD
dev = "cuda"
nh, nkv, d, page, T = 2, 1, 16, 8, 3
pages = torch.zeros(8, 2, nkv, page, d, device=dev)           # 8 pages in memory ...
pool = pages[:4]                                              # ... of which the kernels are told 4
qkv = torch.randn(T, (nh + 2 * nkv) * d, device=dev)
inv_freq = torch.ones(d // 2, device=dev)
token_req = torch.zeros(T, dtype=torch.int32, device=dev)
table = torch.tensor([[1, 6, 2, 0]], dtype=torch.int32, device=dev)   # page 6 is outside the pool of 4
positions = torch.tensor([0, 9, 17], dtype=torch.int32, device=dev)   # position 9 lies in page 6
assert ops.debug_errors() == []
ops.rope_kv(qkv, positions, token_req, table, pool, inv_freq, nh, nkv, d, page)
torch.cuda.synchronize()
found = ops.debug_errors()
assert found == [("elementwise", "a page id outside the pool", 6)], found
assert pages[6].abs().max() == 0 and pages[1].abs().max() > 0 and pages[2].abs().max() > 0   # skipped; the others written
assert ops.debug_errors() == []                                       # reading cleared it

narrow = table[:, :2].contiguous()                                    # position 17 needs a third entry
ops.rope_kv(qkv, positions, token_req, narrow, pages, inv_freq, nh, nkv, d, page)
torch.cuda.synchronize()
assert ops.debug_errors() == [("elementwise", "a position beyond its request's block table", 17)]

out = torch.zeros(T, nh * d, device=dev)
ops.attention_generic(qkv, qkv.stride(0), pool, table, token_req, positions, out, T, nh, nkv, d, page, None, 0.25)
torch.cuda.synchronize()
assert ops.debug_errors() == [("attention_generic", "a page id outside the pool", 6)]
assert torch.isfinite(out).all()

acc = torch.zeros(2, 32, device=dev)
ops.embed(torch.randn(10, 32, device=dev), torch.tensor([3, 12], dtype=torch.int32, device=dev), acc)
torch.cuda.synchronize()
assert ops.debug_errors() == [("elementwise", "a token id outside the vocabulary", 12)]
assert acc[1].abs().max() == 0 and acc[0].abs().max() > 0

try:   # the engine's own read of the error words raises on a failed check
    ops.embed(torch.randn(10, 32, device=dev), torch.tensor([-1], dtype=torch.int32, device=dev), acc[:1])
    ops.raise_on_wait_errors()
    raise SystemExit("no error was raised")
except ops.KernelError as exc:
    assert "debug build" in str(exc) and "-1" in str(exc)
ops.embed(torch.randn(10, 32, device=dev), torch.tensor([5], dtype=torch.int32, device=dev), acc[:1])
ops.raise_on_wait_errors()                                            # and the device is as usable as before
print("debug checks ok")
'''


def test_bad_indices_are_reported_and_skipped():
    proc = _run(["-c", CHECKS], timeout=300)
    assert proc.returncode == 0 and "debug checks ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-3000:]
