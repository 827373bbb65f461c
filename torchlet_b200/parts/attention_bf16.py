"""Choice and planning of the bfloat16 tensor-core attention kernels.  Returns False when
they do not take the sizes (head_dim other than 64 or 128, more than 16 query heads per KV
head); the caller then uses the any-size kernel.

Requests that bring a single token (decode) run in tiles of 16 packed rows with their keys
split over several CTAs, so that a few long requests still fill the GPU
(csrc/attention_mma.cu).  Requests that bring a portion of a prompt run in row tiles planned
here on the host, as the reference plans its prefill tiles
(v10_triton_paged_gqa/layer/gqa.py:163-216): on the tcgen05 kernel (csrc/attention_tc.cu, two
row tiles of whole tokens a CTA) where the page size suits its TMA boxes (8 to 128 tokens,
dividing 128), else in tiles of 64 packed rows on the mma.sync kernel.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops

import functools
import os

ROWS = 64
MIN_KEYS_A_SPLIT = 192  # as MIN_TILES_A_SPLIT x 64 keys in csrc/attention_mma.cu
# TORCHLET_B200_ATTENTION_BESIDE=0: in a mixed step the decode attention waits for the prompt
# portions' kernel to end before it starts (for measurements)
SIDE_BY_SIDE = os.environ.get("TORCHLET_B200_ATTENTION_BESIDE", "1") != "0"


@functools.lru_cache(maxsize=None)
def _sm_count(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def decode_splits(num_requests: int, num_kv_heads: int, max_kv_len: int, device=None) -> int:
    """CTAs the grid of a decode step holds for the keys of one (request, KV head): as many as
    fill ONE wave (three CTAs are resident per SM), at most 64, and no more than the longest
    request the step may meet could use at 192 keys a split (three of the kernel's key tiles; 128
    and 256 were measured: 192 is 0.4-0.9 % of a decode step better at batch 1 to 4).  ``max_kv_len`` is that longest
    length: the step's own longest request, or, where the step is captured in a CUDA graph, the
    engine's length limit.  How many of them a request really uses is decided on the device from
    its own length (csrc/attention_mma.cu, ``effective_splits``), so a grid sized for the limit
    costs a short request nothing but CTAs that leave at once."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    resident = 3 * _sm_count(index)
    room = max(1, resident // max(1, num_requests * num_kv_heads))
    return max(1, min(room, -(-max_kv_len // MIN_KEYS_A_SPLIT), 64))


def prompt_splits(ctas: int, max_kv_len: int, device=None) -> int:
    """Key splits of the tcgen05 prompt attention.  A portion of a prompt beside decoding requests
    has few row tiles (a 512-token portion at 4 KV heads: 60 CTAs for 148 SMs) and each walks the
    whole cached prefix, one key tile after the other.  Where two to four times as many CTAs still
    fit ONE wave, that many share the key tiles of a (row tiles, KV head) and a second kernel
    merges their partial results: 71 -> 51 us for such a portion behind 3,584 cached tokens.  A
    second wave, or a grid that fills the GPU anyway, loses more to the partial results' trip
    through memory than the shorter walk gains (88 CTAs: 74 us whole, 77-90 us split; a whole
    2,048-token prompt: 47 -> 88 us), and so do contexts of fewer than eight key tiles."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    key_tiles = -(-max_kv_len // 128)
    return max(1, min(4, _sm_count(index) // max(1, ctas), key_tiles // 4))


def side_by_side(prompt_splits_chosen: int, prompt_kv_len: int, head_dim: int) -> bool:
    """Whether, in a mixed step, the decode kernel is launched right behind the prompt portions'
    kernel with its wait at its end, so that its CTAs start on the SMs the portions leave idle (few
    row tiles, or the last of several waves) instead of after the portions' last CTA.  Measured on
    the two kernels of one layer, one after the other -> side by side, same key splits
    (``benchmarks.kernels attention --portion``): 32 decoding requests at 2,100 tokens beside a
    1,024-token portion behind 1,024, 8 KV heads of 5 query heads, 108 -> 93 us; beside 2,016 tokens
    at 4 KV heads of 7, 75 -> 72 us; at 2 KV heads of 7 and head_dim 64, 43 -> 38 us; nothing where
    unsplit decode CTAs last as long as the portions' and do not all fit beside them (beside 512
    tokens behind 1,792 at 8 KV heads: 92 us either way).  Where the portions' keys are split, the
    merge of their partial results has to wait for both kernels, which costs 3-5 us: that is taken
    only where the portions' kernel runs some 15 us or more (a 128-key tile takes it about 2.4 us
    at head_dim 128), else short kernels lose (2 KV heads at head_dim 64, four splits: 32 -> 36 us)."""
    if not SIDE_BY_SIDE:
        return False
    if prompt_splits_chosen == 1:
        return True
    tiles = -(-prompt_kv_len // 128)
    return 2.4 * tiles / prompt_splits_chosen * head_dim / 128 >= 15.0


def _plan(ctx, group_size: int, rows_per_tile: int = ROWS):
    """Which requests decode, and the row tiles of the others (uploaded once a step)."""
    key = ("attention_mma", group_size, rows_per_tile)
    plan = ctx.plans.get(key)
    if plan is not None:
        return plan
    indptr = ctx.req_indptr_host
    q_lens = np.diff(indptr)
    if ctx.decode_only:
        plan = {"decode": (None, ctx.num_requests), "prefill": None}
    else:
        decode = np.nonzero(q_lens == 1)[0].astype(np.int32)
        others = np.nonzero(q_lens > 1)[0]
        tile_req, tile_row = [], []
        for r in others:
            rows = int(q_lens[r]) * group_size
            starts = np.arange(0, rows, rows_per_tile, dtype=np.int32)
            tile_req.append(np.full(starts.size, r, dtype=np.int32))
            tile_row.append(starts)
        plan = {"decode": None, "prefill": None}
        if decode.size:
            plan["decode"] = (ctx.upload(decode), int(decode.size))
        if others.size:
            plan["prefill_kv_len"] = int((ctx.kv_before_host[others] + q_lens[others]).max())
            req, row = np.concatenate(tile_req), np.concatenate(tile_row)
            # tiles that see the most keys first: the last CTAs to start are the short ones
            keys_seen = ctx.kv_before_host[req] + row // group_size
            order = np.argsort(-keys_seen, kind="stable")
            req, row = req[order], row[order]
            both = ctx.upload(np.concatenate([req, row]))
            plan["prefill"] = (both[:req.size], both[req.size:], int(req.size))
    ctx.plans[key] = plan
    return plan


def forward(mixer, ctx, qkv, cache, out) -> bool:
    d, nh, nkv = mixer.head_dim, mixer.num_heads, mixer.num_kv_heads
    group = nh // nkv
    if d not in (64, 128) or group > 16 or qkv.stride(0) % 8:
        return False
    # prompt portions: the tcgen05 kernel where it takes the page size, else the mma.sync kernel
    use_tc = (not ctx.decode_only) and ops.attention_tc_supported(d, group, cache.page_size)
    plan = _plan(ctx, group, ops.attention_tc_rows(group) if use_tc else ROWS)
    common = dict(out=out, tokens=ctx.num_tokens, nh=nh, nkv=nkv, d=d, page_size=cache.page_size,
                  window=mixer.window, scale=mixer.scale)
    # A mixed step: the prompt portions first (few CTAs that walk long contexts), the decoding
    # requests' kernel right behind it on the SMs it leaves idle; the two touch different rows.
    merge_portions, beside = None, False
    if plan["prefill"] is not None and use_tc:
        tile_req, tile_row, count = plan["prefill"]
        splits = prompt_splits(count * nkv, plan["prefill_kv_len"], qkv.device)
        beside = plan["decode"] is not None and side_by_side(splits, plan["prefill_kv_len"], d)
        merge_portions = ops.attention_tc(
            qkv, cache.pages, cache.block_table, ctx.req_indptr, ctx.kv_before, tile_req, tile_row, count, out, nh, nkv,
            d, cache.page_size, mixer.window, mixer.scale, splits=splits, token_req=ctx.token_req, defer_merge=beside)
    if plan["decode"] is not None:
        tile_req, count = plan["decode"]
        splits = decode_splits(count, nkv, ctx.max_kv_len, qkv.device)
        ops.attention_mma(qkv, cache.pages, cache.block_table, ctx.req_indptr, ctx.kv_before, tile_req, None,
                          count, rows16=True, splits=splits, late_wait=beside, **common)
    if merge_portions is not None:
        merge_portions()
    if plan["prefill"] is not None and not use_tc:
        tile_req, tile_row, count = plan["prefill"]
        ops.attention_mma(qkv, cache.pages, cache.block_table, ctx.req_indptr, ctx.kv_before, tile_req, tile_row,
                          count, rows16=False, splits=1, **common)
    return True
