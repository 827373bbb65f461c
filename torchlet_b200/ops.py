"""Python entry to the hand-written CUDA kernels.

Every function takes torch CUDA tensors (as containers only), hands raw pointers to
an ``extern "C"`` launcher on torch's current stream, and raises on any error.  There
is no CPU path and no library fallback: a tensor that is not on a CUDA device, a size
a kernel refuses, or a missing library is an error here.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc.build import DEBUG_BUILD, load_library

F32, BF16 = 0, 1
_UNSUPPORTED = 10001


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


_SIGNATURES = {
    "elementwise": {
        "tl_embed": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "tl_rms_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "tl_rope_kv": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "tl_elementwise_debug_error": [c_void_p],
        "tl_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "gemm_simt": {
        "tl_gemm_simt": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_int, c_int, c_void_p],
    },
    "attention_generic": {
        "tl_attention_generic": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "tl_attention_generic_debug_error": [c_void_p],
    },
    "gemm_tc": {
        "tl_gemm_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_longlong,
                       c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p],
        "tl_gemm_tc_plan": [c_int, c_int, c_int, c_void_p, c_void_p],
        "tl_gemm_tc_error": [],
        "tl_gemm_tc_wait_selftest": [c_int, c_void_p],
    },
    "attention_mma": {
        "tl_attention_mma": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                             c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p],
        "tl_attention_mma_error": [],
        "tl_attention_mma_debug_error": [c_void_p],
    },
    "decode_fused": {
        "tl_finish_qkv_rope": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "tl_decode_fused_debug_error": [c_void_p],
        "tl_finish_accum_norm": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                 c_void_p],
    },
    "attention_tc": {
        "tl_attention_tc": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_float,
                            c_int, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p],
        "tl_attention_tc_merge": [c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                  c_longlong, c_void_p],
        "tl_attention_tc_error": [],
        "tl_attention_tc_rows": [c_int],
    },
    "slots": {
        "tl_slot_gather": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "tl_slot_advance": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "tl_slot_command_words": [c_int, c_int],
        "tl_slot_record_rows": [],
        "tl_slots_debug_error": [c_void_p],
    },
    "sampling": {
        "tl_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_longlong, c_void_p],
    },
}

_functions: dict[str, ctypes._CFuncPtr] = {}


def _fn(library: str, name: str):
    fn = _functions.get(name)
    if fn is None:
        lib = load_library(library)
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[library][name]
        fn.restype = c_longlong if name.endswith("_plan") else c_int
        _functions[name] = fn
    return fn


launch_count = 0  # kernels launched through this module (graph replays are counted by the runner)


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += kernels
        return
    if code == _UNSUPPORTED:
        raise KernelError(f"{what}: sizes or types not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The handle of the current CUDA stream of the current device.  (Asked through the raw
    accessor where torch has one: building a ``torch.cuda.Stream`` object for every launch
    was a third of the host's time in a step of small kernels.)"""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


# ------------------------------------------------------------------ wrappers
def embed(table: torch.Tensor, ids: torch.Tensor, acc: torch.Tensor) -> None:
    """acc[t] = float32(table[ids[t]]);  ids int32 [T], acc float32 [T, hidden]."""
    _need_cuda(table, ids, acc)
    tokens, hidden = acc.shape
    assert ids.dtype == torch.int32 and acc.dtype == torch.float32 and acc.is_contiguous()
    assert table.is_contiguous() and table.shape[1] == hidden
    code = _fn("elementwise", "tl_embed")(
        table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), acc.data_ptr(), tokens, hidden,
        table.shape[0], _stream())
    _check(code, "embed")


def rms_norm(acc: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, rows=None) -> None:
    """out[r] = rmsnorm(acc[rows[r] or r]) * weight;  acc float32, weight float32."""
    _need_cuda(acc, weight, out, rows)
    hidden = acc.shape[1]
    num_rows = out.shape[0]
    assert acc.dtype == torch.float32 and weight.dtype == torch.float32
    assert acc.is_contiguous() and out.is_contiguous() and out.shape[1] == hidden
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= num_rows)
    code = _fn("elementwise", "tl_rms_norm")(
        acc.data_ptr(), weight.data_ptr(), _ptr(rows), out.data_ptr(), dtype_code(out.dtype), num_rows,
        hidden, float(eps), _stream())
    _check(code, "rms_norm")


def rope_kv(qkv, positions, token_req, block_table, pages, inv_freq, nh, nkv, d, page_size, write_kv=True):
    """Rotate q (in place) and k by position, write k and v into cache pages."""
    _need_cuda(qkv, positions, token_req, block_table, pages, inv_freq)
    tokens = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d
    assert pages.dtype == qkv.dtype and inv_freq.dtype == torch.float32 and inv_freq.numel() == d // 2
    code = _fn("elementwise", "tl_rope_kv")(
        qkv.data_ptr(), dtype_code(qkv.dtype), positions.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], pages.data_ptr(), inv_freq.data_ptr(), tokens, nh, nkv,
        d, page_size, 1 if write_kv else 0, pages.shape[0], _stream())
    _check(code, "rope_kv")


def store_kv(qkv, positions, token_req, block_table, pages, nh, nkv, d, page_size) -> None:
    """Write the k and v heads of the fused ``qkv`` rows to the cache pages, unchanged (for a mixer
    whose position encoding, if any, does not store them itself)."""
    _need_cuda(qkv, positions, token_req, block_table, pages)
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d and pages.dtype == qkv.dtype
    code = _fn("elementwise", "tl_rope_kv")(
        qkv.data_ptr(), dtype_code(qkv.dtype), positions.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], pages.data_ptr(), None, qkv.shape[0], nh, nkv,
        d, page_size, 1, pages.shape[0], _stream())
    _check(code, "store_kv")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need_cuda(gate_up, out)
    tokens, inter = out.shape
    assert gate_up.shape == (tokens, 2 * inter) and gate_up.is_contiguous() and out.is_contiguous()
    assert gate_up.dtype == out.dtype
    code = _fn("elementwise", "tl_swiglu")(
        gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), tokens, inter, _stream())
    _check(code, "swiglu")


def gemm_simt(x, w, out, bias=None, accumulate=False) -> None:
    """out (+)= x @ w.T + bias on CUDA cores, float32 accumulation in ascending k."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and x.dtype == w.dtype
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == N)
    assert not accumulate or out.dtype == torch.float32
    code = _fn("gemm_simt", "tl_gemm_simt")(
        x.data_ptr(), w.data_ptr(), dtype_code(x.dtype), _ptr(bias), out.data_ptr(), dtype_code(out.dtype),
        1 if accumulate else 0, M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream())
    _check(code, "gemm_simt")


def attention_generic(q, q_stride, pages, block_table, token_req, positions, out, tokens, nh, nkv, d,
                      page_size, window, scale) -> None:
    """Paged causal GQA attention, one warp per (token, head); q may be a view into qkv."""
    _need_cuda(q, pages, block_table, token_req, positions, out)
    assert q.dtype == pages.dtype == out.dtype and out.is_contiguous()
    code = _fn("attention_generic", "tl_attention_generic")(
        q.data_ptr(), q_stride, pages.data_ptr(), dtype_code(q.dtype), block_table.data_ptr(),
        block_table.shape[1], token_req.data_ptr(), positions.data_ptr(), out.data_ptr(), out.stride(0),
        tokens, nh, nkv, d, page_size, int(window or 0), float(scale), pages.shape[0], _stream())
    _check(code, "attention_generic")


def sample(logits, out, temperature=None, seed=None, counter=None) -> None:
    """out[r] = argmax(logits[r]) or a seeded draw from softmax(logits[r] / temperature[r])."""
    _need_cuda(logits, out, temperature, seed, counter)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seed.dtype == torch.int64 and counter.dtype == torch.int32
    chunks = -(-vocab // 8192)
    scratch = _workspace(("sample", logits.device), rows * chunks * 8) if chunks > 1 else None
    code = _fn("sampling", "tl_sample")(
        logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(seed), _ptr(counter),
        out.data_ptr(), _ptr(scratch), scratch.numel() * 4 if scratch is not None else 0, _stream())
    _check(code, "sample", 2 if chunks > 1 else 1)


# ---------------------------------------------------------------- slot records
def slot_record_rows() -> int:
    return _fn("slots", "tl_slot_record_rows")()


def slot_command_words(lanes: int, capacity: int) -> int:
    """int32 words of the command block of a decode step (csrc/slots.cu)."""
    return _fn("slots", "tl_slot_command_words")(lanes, capacity)


def slot_gather(command, lanes: int, groups: int, max_slots: int, width: int, page_size: int, records, slot_tables,
                token, position, kv_before, slot, seed, temperature, counter, lane_tables) -> None:
    """From the slot records (and the command block's news) to the lane-indexed words a decode
    step's kernels read: tokens, positions, sampling words, block-table rows."""
    _need_cuda(command, records, slot_tables, token, position, kv_before, slot, seed, temperature, counter, lane_tables)
    assert records.dtype == torch.int32 and records.is_contiguous() and records.shape[1] == max_slots
    assert seed.dtype == torch.int64 and temperature.dtype == torch.float32
    code = _fn("slots", "tl_slot_gather")(
        command.data_ptr(), lanes, groups, max_slots, width, page_size, records.data_ptr(), _ptr(slot_tables),
        token.data_ptr(), position.data_ptr(), kv_before.data_ptr(), slot.data_ptr(), seed.data_ptr(),
        temperature.data_ptr(), counter.data_ptr(), _ptr(lane_tables), _stream())
    _check(code, "slot_gather")


def slot_advance(command, lanes: int, max_slots: int, sampled, records) -> None:
    """After sampling: each live lane's slot takes the sampled token, position + 1, counter + 1."""
    _need_cuda(command, sampled, records)
    code = _fn("slots", "tl_slot_advance")(command.data_ptr(), lanes, max_slots, sampled.data_ptr(),
                                           records.data_ptr(), _stream())
    _check(code, "slot_advance")


# ------------------------------------------------------- tensor-core products
EPI_STORE_BF16, EPI_ACCUM_F32, EPI_SWIGLU_BF16, EPI_STORE_F32 = 0, 1, 2, 3
_workspaces: dict = {}
_outgrown: list = []  # kept alive: captured CUDA graphs may still hold their addresses


def _workspace(device, nbytes: int) -> torch.Tensor:
    """A float32 scratch buffer per device that only grows (split-K partial sums)."""
    ws = _workspaces.get(device)
    if ws is None or ws.numel() * 4 < nbytes:
        if ws is not None:
            _outgrown.append(ws)
        where = device[1] if isinstance(device, tuple) else device
        ws = torch.empty(max(nbytes // 4 + 1, 1 << 22), dtype=torch.float32, device=where)
        _workspaces[device] = ws
    return ws


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Sizes the tcgen05 product takes: K and both row strides multiples of 8 elements,
    16-byte aligned bases."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(1) == 1 and w.stride(1) == 1)


# The step context that holds unfinished partial sums in the shared workspace, if any; it
# is asked to finish them before another product overwrites the workspace.
workspace_holder = None


def _release_workspace() -> None:
    if workspace_holder is not None:
        workspace_holder.flush_pending()


_plans: dict = {}  # (M, N, K) -> (workspace bytes, swapped orientation, splits): fixed for a process


def _gemm_plan(M: int, N: int, K: int) -> tuple:
    plan = _plans.get((M, N, K))
    if plan is None:
        swap, splits = ctypes.c_int(0), ctypes.c_int(0)
        need = _fn("gemm_tc", "tl_gemm_tc_plan")(M, N, K, ctypes.byref(swap), ctypes.byref(splits))
        plan = _plans[(M, N, K)] = (need, bool(swap.value), splits.value)
    return plan


def gemm_tc(x, w, out, bias=None, epilogue=EPI_STORE_BF16, cta_pairs=None) -> None:
    """out (+)= x @ w.T (+ bias) on the tcgen05 tensor cores; see csrc/gemm_tc.cu.
    ``cta_pairs``: for many tokens, True forces the kernel in which two CTAs share one 256-row
    MMA, False the single-CTA kernel; None lets the library choose (pairs where their 256-row tiles cover no more rows than 128-row tiles)."""
    _need_cuda(x, w, out, bias)
    _release_workspace()
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1
    want = torch.bfloat16 if epilogue in (EPI_STORE_BF16, EPI_SWIGLU_BF16) else torch.float32
    assert out.dtype == want and out.shape == (M, N // 2 if epilogue == EPI_SWIGLU_BF16 else N)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == N)
    need, _, splits = _gemm_plan(M, N, K)
    ws = _workspace(x.device, need) if need else None
    kernels = 2 if need and splits > 1 else 1  # several splits: product + finishing pass
    code = _fn("gemm_tc", "tl_gemm_tc")(
        x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), out.stride(0), epilogue, M, N, K, x.stride(0),
        w.stride(0), _ptr(ws), ws.numel() * 4 if ws is not None else 0, {None: 0, True: 2, False: 3}[cta_pairs], None,
        _stream())
    _check(code, "gemm_tc", kernels)


def gemm_tc_deferred(x, w):
    """The product x @ w.T left as float32 partial sums ``[splits, M, N]`` for a fused
    finishing kernel.  Returns (partials, splits), or None when the sizes run in a
    kernel that writes its output directly (many tokens, no K splits)."""
    _need_cuda(x, w)
    _release_workspace()
    M, K = x.shape
    N = w.shape[0]
    need, swap, planned = _gemm_plan(M, N, K)
    if not swap and planned <= 1:
        return None
    ws = _workspace(x.device, need)
    splits = ctypes.c_int(0)
    code = _fn("gemm_tc", "tl_gemm_tc")(
        x.data_ptr(), w.data_ptr(), None, None, 0, EPI_STORE_F32, M, N, K, x.stride(0), w.stride(0), ws.data_ptr(),
        ws.numel() * 4, 1, ctypes.byref(splits), _stream())
    _check(code, "gemm_tc (deferred)")
    return ws, splits.value


def finish_qkv_rope(partials, splits, bias, qkv, positions, token_req, block_table, pages, inv_freq, nh, nkv, d,
                    page_size, write_kv=True) -> None:
    """Sum the qkv product's splits (+ bias), rotate q and k, store q to ``qkv`` and k, v to pages."""
    _need_cuda(partials, bias, qkv, positions, token_req, block_table, pages, inv_freq)
    assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d
    code = _fn("decode_fused", "tl_finish_qkv_rope")(
        partials.data_ptr(), splits, _ptr(bias), qkv.data_ptr(), positions.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], pages.data_ptr(), inv_freq.data_ptr(), qkv.shape[0], nh, nkv,
        d, page_size, 1 if write_kv else 0, pages.shape[0], _stream())
    _check(code, "finish_qkv_rope")


def finish_accum_norm(partials, splits, bias, acc, weight=None, eps=0.0, out=None) -> None:
    """acc += sum of the splits (+ bias); with ``out``: out = rmsnorm(acc) * weight (bfloat16)."""
    _need_cuda(partials, bias, acc, weight, out)
    tokens, hidden = acc.shape
    assert acc.dtype == torch.float32 and acc.is_contiguous()
    assert out is None or (out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == acc.shape)
    code = _fn("decode_fused", "tl_finish_accum_norm")(
        partials.data_ptr(), splits, _ptr(bias), acc.data_ptr(), _ptr(weight), _ptr(out), tokens, hidden,
        float(eps), _stream())
    _check(code, "finish_accum_norm")


def gemm_tc_error() -> int:
    """0, or the code a bounded wait in a tensor-core kernel left when it gave up
    (1 producer, 2 MMA issuer, 3 epilogue).  Reading clears it."""
    return _fn("gemm_tc", "tl_gemm_tc_error")()


def wait_selftest(code: int = 99) -> None:
    """Launches one block whose bounded wait runs out (nothing ever arrives at its barrier; the
    limit is 2^16 cycles) and that then returns normally: ``gemm_tc_error()`` afterwards gives
    ``code`` and ``raise_on_wait_errors()`` raises.  Nothing faults or hangs; for tests."""
    _check(_fn("gemm_tc", "tl_gemm_tc_wait_selftest")(code, _stream()), "wait_selftest")


_arrival_counters: dict = {}
_outgrown_counters: list = []  # kept alive: captured CUDA graphs may still hold their addresses


def _arrivals(device, count: int) -> torch.Tensor:
    """Per device, ints that are zero between launches: the decode attention counts the key
    splits of a (request, KV head) that have finished; the last one merges and zeroes its counter."""
    counters = _arrival_counters.get(device)
    if counters is None or counters.numel() < count:
        if counters is not None:
            _outgrown_counters.append(counters)
        counters = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _arrival_counters[device] = counters
    return counters


# TORCHLET_B200_DECODE_MERGE=kernel: a second kernel merges the key splits (for measurements)
_merge_in_kernel = os.environ.get("TORCHLET_B200_DECODE_MERGE", "") != "kernel"


def attention_mma(qkv, pages, block_table, req_indptr, kv_before, tile_req, tile_row, tiles, out, tokens, nh, nkv,
                  d, page_size, window, scale, rows16: bool, splits: int = 1, late_wait: bool = False) -> None:
    """Tensor-core paged attention (csrc/attention_mma.cu).  ``tile_req``/``tile_row`` None:
    tile i is request i from its first packed row.  With ``splits`` > 1 every tile is a request
    that brings one token; only those tokens' rows of ``out`` are written.  ``splits`` is the
    number of CTAs the grid holds for a request's keys; the kernel uses as many as the request's
    own length warrants.  ``late_wait`` (16-row tiles): the launch just before this one on the
    stream was ``attention_tc`` for the other requests of the same step; this grid starts beside
    it and waits for it at its end instead of at its start."""
    _need_cuda(qkv, pages, block_table, req_indptr, kv_before, tile_req, tile_row, out)
    assert qkv.dtype == pages.dtype == out.dtype == torch.bfloat16
    # key splits: float32 partial results of every (decode tile, head, split); the split that finishes last merges
    need = tiles * nh * splits * (d + 2) * 4 if splits > 1 else 0
    ws = _workspace(("attention", qkv.device), need) if need else None
    # up to 16 splits the last split to finish merges them inside the kernel (one round of loads;
    # measured -1 % of a decode step at batch 8 to 32); more are merged by a second kernel, whose
    # many small CTAs do better than one CTA's two rounds (batch 1 at 4,096 tokens: 32 splits)
    arrivals = _arrivals(qkv.device, tiles * nkv) if need and _merge_in_kernel and splits <= 16 else None
    code = _fn("attention_mma", "tl_attention_mma")(
        qkv.data_ptr(), qkv.stride(0), pages.data_ptr(), pages.shape[0], block_table.data_ptr(),
        block_table.shape[1], req_indptr.data_ptr(), kv_before.data_ptr(), _ptr(tile_req), _ptr(tile_row), tiles,
        out.data_ptr(), out.stride(0), tokens, nh, nkv, d, page_size, int(window or 0), float(scale),
        1 if rows16 else 0, splits,
        _ptr(ws), ws.numel() * 4 if ws is not None else 0, _ptr(arrivals), 1 if late_wait else 0, _stream())
    _check(code, "attention_mma", 2 if splits > 1 and arrivals is None else 1)


def attention_tc_rows(group: int) -> int:
    """Packed rows a tile of the tcgen05 attention kernel holds for ``group`` heads a KV head."""
    return _fn("attention_tc", "tl_attention_tc_rows")(group)


def attention_tc_supported(d: int, group: int, page_size: int) -> bool:
    return d in (64, 128) and 1 <= group <= 128 and 8 <= page_size <= 128 and 128 % page_size == 0


def attention_tc(qkv, pages, block_table, req_indptr, kv_before, tile_req, tile_row, tiles, out, nh, nkv, d,
                 page_size, window, scale, splits: int = 1, token_req=None, defer_merge: bool = False):
    """Prompt-portion attention on tcgen05 (csrc/attention_tc.cu): tiles of packed rows
    (``tile_row`` multiples of ``attention_tc_rows(nh // nkv)``) that cover every request of the
    step with more than one token.  ``splits`` > 1: that many CTAs share the key tiles of each
    (row tiles, KV head) and a second kernel merges them (``token_req``: each token's request).
    ``defer_merge``: that second kernel is not launched; the call returns a function that launches
    it (None when there is nothing to merge), so that the decode attention may run between the two.
    The partial results have a workspace of their own."""
    _need_cuda(qkv, pages, block_table, req_indptr, kv_before, tile_req, tile_row, out, token_req)
    assert qkv.dtype == pages.dtype == out.dtype == torch.bfloat16 and pages.is_contiguous()
    tokens = qkv.shape[0]
    need = tokens * nh * splits * (d + 2) * 4 if splits > 1 else 0
    ws = _workspace(("attention_tc", qkv.device), need) if need else None
    ws_bytes = ws.numel() * 4 if ws is not None else 0
    defer = defer_merge and splits > 1
    code = _fn("attention_tc", "tl_attention_tc")(
        qkv.data_ptr(), qkv.stride(0), pages.data_ptr(), pages.shape[0], block_table.data_ptr(),
        block_table.shape[1], req_indptr.data_ptr(), kv_before.data_ptr(), tile_req.data_ptr(), tile_row.data_ptr(),
        tiles, out.data_ptr(), out.stride(0), nh, nkv, d, page_size, int(window or 0), float(scale), splits,
        _ptr(token_req), tokens, _ptr(ws), ws_bytes, 1 if defer else 0, _stream())
    _check(code, "attention_tc", 2 if splits > 1 and not defer else 1)
    if not defer:
        return None

    def merge() -> None:
        code = _fn("attention_tc", "tl_attention_tc_merge")(
            req_indptr.data_ptr(), out.data_ptr(), out.stride(0), nh, d, splits, token_req.data_ptr(), tokens,
            ws.data_ptr(), ws_bytes, _stream())
        _check(code, "attention_tc_merge", 1)

    return merge


def attention_mma_error() -> int:
    """0, or the code a bounded wait of the decode attention's TMA loader left.  Reading clears it
    (and the arrival counters, which a kernel that gave up may have left half counted)."""
    code = _fn("attention_mma", "tl_attention_mma_error")()
    if code:
        for counters in _arrival_counters.values():
            counters.zero_()
    return code


def attention_tc_error() -> int:
    """0, or the code a bounded wait in the tcgen05 attention kernel left when it gave up."""
    return _fn("attention_tc", "tl_attention_tc_error")()


_DEBUG_CODES = {1: "a token id outside the vocabulary", 2: "a position beyond its request's block table",
                3: "a page id outside the pool", 4: "a slot outside the slot range"}


def debug_errors() -> list:
    """What the debug build's index checks have caught since the last call: (library, meaning,
    offending value) for every loaded library whose check failed; reading clears.  Always empty
    in the ordinary build (``TORCHLET_B200_DEBUG`` unset), whose kernels carry no checks."""
    found = []
    for library in ("elementwise", "attention_generic", "attention_mma", "decode_fused", "slots"):
        if any(name in _functions for name in _SIGNATURES[library]):
            value = ctypes.c_int(0)
            code = _fn(library, f"tl_{library}_debug_error")(ctypes.byref(value))
            if code:
                found.append((library, _DEBUG_CODES.get(code, f"code {code}"), value.value))
    return found


def raise_on_wait_errors() -> None:
    """Raises if a bounded wait inside a tensor-core kernel has given up since the last call
    (the kernel then ran to its end with whatever it had, so its output is not to be used), or,
    in the debug build, if an index check inside a kernel has failed.
    Only libraries that are loaded are asked.  The read is a blocking copy on the default
    stream, so it sees every kernel launched before it."""
    for library, read in (("gemm_tc", gemm_tc_error), ("attention_tc", attention_tc_error),
                          ("attention_mma", attention_mma_error)):
        if any(name in _functions for name in _SIGNATURES[library]):
            code = read()
            if code:
                raise KernelError(f"{library}: a bounded wait gave up inside a kernel (code {code}); "
                                  "the results of this step are invalid")
    if DEBUG_BUILD:
        for library, meaning, value in debug_errors():
            raise KernelError(f"{library} (debug build): {meaning}: {value}; the access was skipped, "
                              "the results of this step are invalid")