"""The sampling entry point that allocates nothing (csrc/sampling_static.h), called through
its exported C symbol and compared with the ordinary entry point, which takes its scratch
from the caller.  It serves callers that may not allocate device memory when they need a
token (inside a stream capture, or where another component owns the memory pool), so the
test passes only inputs and outputs and checks two calls in a row: the second call finds
the fixed scratch array still holding the first call's contents and must not be misled by
them.  Collected last on purpose (a failure here leaves every other test already run)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
TOO_LARGE = 10002


def _static_entry():
    from torchlet_b200.csrc.build import load_library

    fn = load_library("sampling").tl_sample_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def _call(fn, logits, out, temperature=None, seed=None, counter=None):
    ptr = lambda t: None if t is None else t.data_ptr()
    return fn(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], ptr(temperature), ptr(seed),
              ptr(counter), out.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from torchlet_b200 import ops

    fn = _static_entry()
    dev = "cuda"
    generator = torch.Generator(device="cpu")
    cases = [(7, 20011, 1), (3, 50000, 2)]  # (rows, vocabulary, seed): several chunks a row, the second call differs
    for rows, vocab, s in cases:
        logits = (torch.randn(rows, vocab, generator=generator.manual_seed(s)) * 3).to(dev)
        temperature = torch.tensor([0.0, 0.8, 1.3, 0.0, 0.5, 2.0, 1.0][:rows], device=dev)
        seed = torch.arange(rows, dtype=torch.int64, device=dev) + 11 * s
        counter = torch.arange(rows, dtype=torch.int32, device=dev) * 3
        for sampling in (None, (temperature, seed, counter)):
            want = torch.full((rows,), -1, dtype=torch.int32, device=dev)
            got = torch.full((rows,), -2, dtype=torch.int32, device=dev)
            args = sampling or (None, None, None)
            ops.sample(logits, want, *args)
            assert _call(fn, logits, got, *args) == 0
            torch.cuda.synchronize()
            assert torch.equal(got, want)  # the same kernels and the same order of comparisons: identical tokens
            if sampling is None:
                assert torch.equal(got.long().cpu(), logits.cpu().argmax(-1))


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    fn = _static_entry()
    rows, vocab = 600, 500_000  # 600 * ceil(500000 / 8192) = 37200 partial results > 32768
    logits = torch.zeros(1, vocab, device="cuda").expand(rows, vocab)  # stride 0 rows: no large allocation
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    assert _call(fn, logits, out) == TOO_LARGE
    assert _call(fn, logits[:1], out[:1]) == 0  # a size that fits still works afterwards
    torch.cuda.synchronize()
    assert int(out[0]) == 0


def test_static_scratch_entry_point_refuses_a_temperature_without_seed_or_counter():
    """Return codes only: a refused call launches nothing."""
    fn = _static_entry()
    logits = torch.zeros(2, 100, device="cuda")
    out = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    temperature = torch.ones(2, device="cuda")
    seed = torch.zeros(2, dtype=torch.int64, device="cuda")
    counter = torch.zeros(2, dtype=torch.int32, device="cuda")
    unsupported = 10001
    assert _call(fn, logits, out, temperature, None, None) == unsupported
    assert _call(fn, logits, out, temperature, seed, None) == unsupported
    assert _call(fn, logits, out, temperature, None, counter) == unsupported
    torch.cuda.synchronize()
    assert out.tolist() == [-1, -1]  # nothing ran
    assert _call(fn, logits, out, temperature, seed, counter) == 0
    torch.cuda.synchronize()
    assert all(0 <= t < 100 for t in out.tolist())
