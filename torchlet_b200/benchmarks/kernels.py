"""Single kernels at chosen sizes, timed with CUDA events (also the small cases that are
profiled with ncu for ``profiles/``).

    python -m torchlet_b200.benchmarks.kernels gemm --m 8 --n 37888 --k 3584 --epilogue swiglu
    python -m torchlet_b200.benchmarks.kernels attention --batch 8 --context 4096 --q-len 1
    python -m torchlet_b200.benchmarks.kernels attention --batch 1 --context 0 --q-len 2048
    python -m torchlet_b200.benchmarks.kernels attention --batch 32 --context 2100 --portion 2016 --heads 40 --kv-heads 8

Weights rotate through several copies so that together they exceed the 126 MB L2; each
line reports the mean time of ``--iters`` launches after ``--warmup``.
"""
from __future__ import annotations

import argparse

import torch

from .. import ops

EPILOGUES = {"bf16": ops.EPI_STORE_BF16, "accum": ops.EPI_ACCUM_F32, "swiglu": ops.EPI_SWIGLU_BF16,
             "f32": ops.EPI_STORE_F32}


USE_GRAPH = False  # --graph: the timed launches are replayed from one CUDA graph (no host time between them)


def _time(fn, iters: int, warmup: int) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if USE_GRAPH:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                fn(warmup + i)
        graph.replay()
        torch.cuda.synchronize()
        begin.record()
        graph.replay()
        end.record()
    else:
        begin.record()
        for i in range(iters):
            fn(warmup + i)
        end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / iters


def bench_gemm(args) -> None:
    M, N, K = args.m, args.n, args.k
    epilogue = EPILOGUES[args.epilogue]
    copies = max(1, min(8, -(-(200 << 20) // (N * K * 2))))  # > L2 in total
    generator = torch.Generator(device="cuda").manual_seed(0)
    weights = [(torch.randn(N, K, device="cuda", generator=generator) * 0.02).bfloat16() for _ in range(copies)]
    x = (torch.randn(M, K, device="cuda", generator=generator)).bfloat16()
    out_cols = N // 2 if args.epilogue == "swiglu" else N
    out = torch.zeros(M, out_cols, device="cuda", dtype=torch.bfloat16 if args.epilogue in ("bf16", "swiglu") else torch.float32)
    ms = _time(lambda i: ops.gemm_tc(x, weights[i % copies], out, None, epilogue, cta_pairs={"auto": None, "on": True, "off": False}[args.pairs]), args.iters,
               args.warmup)
    flops, weight_bytes = 2.0 * M * N * K, N * K * 2
    print(f"gemm M={M} N={N} K={K} epilogue={args.epilogue}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.1f} TFLOP/s, "
          f"weights {weight_bytes / ms / 1e6:.0f} GB/s, wait-error {ops.gemm_tc_error()}")


def bench_attention(args) -> None:
    from ..parts.attention_bf16 import ROWS, decode_splits

    nh, nkv, d, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    n, before, q_len = args.batch, args.context, args.q_len
    total = before + q_len
    width = -(-total // page)
    pages = (torch.randn(n * width + 1, 2, nkv, page, d, device="cuda") * 0.5).bfloat16()
    table = (torch.randperm(n * width, device="cuda").to(torch.int32) + 1).view(n, width).contiguous()
    qkv = torch.randn(n * q_len, (nh + 2 * nkv) * d, device="cuda").bfloat16()
    out = torch.zeros(n * q_len, nh * d, device="cuda", dtype=torch.bfloat16)
    indptr = torch.arange(0, (n + 1) * q_len, q_len, dtype=torch.int32, device="cuda")
    kv_before = torch.full((n,), before, dtype=torch.int32, device="cuda")
    scale = d ** -0.5
    group = nh // nkv
    if q_len == 1:
        splits = args.splits or decode_splits(n, nkv, total)
        run = lambda i: ops.attention_mma(qkv, pages, table, indptr, kv_before, None, None, n, out, n, nh, nkv, d, page,
                                          None, scale, rows16=True, splits=splits)
        kv_bytes = n * total * 2 * nkv * d * 2
        what = f"decode splits={splits}"
    elif args.kernel == "tc" and ops.attention_tc_supported(d, group, page):
        rows = ops.attention_tc_rows(group)
        tiles = sorted(((r, s) for r in range(n) for s in range(0, q_len * group, rows)), key=lambda t: -t[1])
        tile_req = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
        tile_row = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
        from ..parts.attention_bf16 import prompt_splits

        splits = args.splits or prompt_splits(len(tiles) * nkv, total)
        token_req = torch.arange(n, dtype=torch.int32, device="cuda").repeat_interleave(q_len)
        run = lambda i: ops.attention_tc(qkv, pages, table, indptr, kv_before, tile_req, tile_row, len(tiles), out,
                                         nh, nkv, d, page, None, scale, splits=splits, token_req=token_req)
        kv_bytes = n * total * 2 * nkv * d * 2
        what = f"prompt (tcgen05) tiles={len(tiles)} key splits={splits}"
    else:
        tiles = [(r, s) for r in range(n) for s in range(0, q_len * group, ROWS)]
        tile_req = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
        tile_row = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
        run = lambda i: ops.attention_mma(qkv, pages, table, indptr, kv_before, tile_req, tile_row, len(tiles), out,
                                          n * q_len, nh, nkv, d, page, None, scale, rows16=False)
        kv_bytes = n * total * 2 * nkv * d * 2
        what = f"prompt tiles={len(tiles)}"
    ms = _time(run, args.iters, args.warmup)
    flops = 4.0 * n * nh * d * (q_len * before + q_len * (q_len + 1) / 2)
    print(f"attention batch={n} context={before} q_len={q_len} heads={nh}/{nkv} d={d} {what}: {ms * 1e3:.1f} us, "
          f"{flops / ms / 1e9:.1f} TFLOP/s, KV {kv_bytes / ms / 1e6:.0f} GB/s")


def bench_mixed_attention(args) -> None:
    """The two attention kernels of a mixed step (``--batch`` requests that decode at
    ``--context`` tokens beside one ``--portion``-token portion of a prompt behind
    ``--portion-context`` cached tokens): the decode kernel after the portion's kernel has ended,
    and beside it (its wait moved to its end), with the engine's key splits."""
    from ..parts.attention_bf16 import decode_splits, prompt_splits, side_by_side

    nh, nkv, d, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    n, before, portion, behind = args.batch, args.context, args.portion, args.portion_context
    group = nh // nkv
    lengths = [before + 1] * n + [behind + portion]
    widths = [-(-length // page) for length in lengths]
    num_pages = sum(widths) + 1
    pages = (torch.randn(num_pages, 2, nkv, page, d, device="cuda") * 0.5).bfloat16()
    order = torch.randperm(num_pages - 1, device="cuda").to(torch.int32) + 1
    table = torch.zeros(n + 1, max(widths), dtype=torch.int32, device="cuda")
    start = 0
    for i, w in enumerate(widths):
        table[i, :w] = order[start:start + w]
        start += w
    tokens = n + portion
    qkv = torch.randn(tokens, (nh + 2 * nkv) * d, device="cuda").bfloat16()
    out = torch.zeros(tokens, nh * d, device="cuda", dtype=torch.bfloat16)
    to = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    indptr, kv_before = to(list(range(n + 1)) + [tokens]), to([before] * n + [behind])
    rows = ops.attention_tc_rows(group)
    starts = list(range(0, portion * group, rows))[::-1]  # the tiles that see the most keys first
    tile_req, tile_row, decoders = to([n] * len(starts)), to(starts), to(list(range(n)))
    token_req = to(list(range(n)) + [n] * portion)
    scale = d ** -0.5
    p_splits = prompt_splits(len(starts) * nkv, behind + portion)
    d_splits = decode_splits(n, nkv, max(lengths))

    def run(beside: bool) -> None:
        merge = ops.attention_tc(qkv, pages, table, indptr, kv_before, tile_req, tile_row, len(starts), out, nh, nkv, d,
                                 page, None, scale, splits=p_splits, token_req=token_req, defer_merge=beside)
        ops.attention_mma(qkv, pages, table, indptr, kv_before, decoders, None, n, out, tokens, nh, nkv, d, page, None,
                          scale, rows16=True, splits=d_splits, late_wait=beside)
        if merge is not None:
            merge()

    spacer = torch.zeros(1024, device="cuda")  # an ordinary launch between iterations: nothing overlaps across them

    def timed(fn) -> float:
        return _time(lambda i: (spacer.add_(1), fn()), args.iters, args.warmup)

    empty = timed(lambda: None)
    in_turn, beside = timed(lambda: run(False)) - empty, timed(lambda: run(True)) - empty
    print(f"mixed attention: {n} decoding at {before} beside {portion} tokens behind {behind}, heads={nh}/{nkv} d={d}, "
          f"portion CTAs {len(starts) * nkv} x {p_splits} key splits, decode key splits {d_splits}: in turn "
          f"{in_turn * 1e3:.1f} us, side by side {beside * 1e3:.1f} us (the engine's choice: "
          f"{'side by side' if side_by_side(p_splits, behind + portion, d) else 'in turn'})")


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = parser.add_subparsers(dest="what", required=True)
    gemm = sub.add_parser("gemm")
    gemm.add_argument("--m", type=int, default=8)
    gemm.add_argument("--n", type=int, default=37888)
    gemm.add_argument("--k", type=int, default=3584)
    gemm.add_argument("--epilogue", choices=sorted(EPILOGUES), default="swiglu")
    gemm.add_argument("--pairs", choices=["auto", "on", "off"], default="auto",
                      help="many tokens: the CTA-pair kernel (cta_group::2), the single-CTA kernel, or the library's choice")
    attention = sub.add_parser("attention")
    attention.add_argument("--batch", type=int, default=8)
    attention.add_argument("--context", type=int, default=4096)
    attention.add_argument("--q-len", type=int, default=1)
    attention.add_argument("--heads", type=int, default=28)
    attention.add_argument("--kv-heads", type=int, default=4)
    attention.add_argument("--head-dim", type=int, default=128)
    attention.add_argument("--page-size", type=int, default=16)
    attention.add_argument("--splits", type=int, default=0,
                           help="CTAs that share the key tiles of a (request or row tiles, KV head) (0: the engine's choice)")
    attention.add_argument("--kernel", choices=["tc", "mma"], default="tc",
                           help="prompt portions: tcgen05 kernel (head_dim 128) or the mma.sync kernel")
    attention.add_argument("--portion", type=int, default=0,
                           help="a mixed step: the --batch requests decode beside one portion of this many prompt tokens")
    attention.add_argument("--portion-context", type=int, default=0, help="cached tokens before that portion")
    for p in (gemm, attention):
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--warmup", type=int, default=3)
        p.add_argument("--graph", action="store_true",
                       help="replay the timed launches from one CUDA graph (for kernels shorter than a launch costs the host)")
    args = parser.parse_args(argv)
    global USE_GRAPH
    USE_GRAPH = args.graph
    if args.what == "attention" and args.portion > 0:
        bench_mixed_attention(args)
        return 0
    {"gemm": bench_gemm, "attention": bench_attention}[args.what](args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
