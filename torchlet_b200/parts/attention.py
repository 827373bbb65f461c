"""Grouped-query attention mixer over a paged cache.

q = x Wq^T + bq, k = x Wk^T + bk, v = x Wv^T + bv; position encoding on q and k (if the
layer has one; ``positions`` may be absent); keys
and values of the step's tokens go to the request's pages; every token attends to the
keys of its request at positions <= its own (and within ``window`` of it, if set), query
head h reading KV head h // (heads / kv_heads); softmax(q.k * scale) in float32; the
heads' outputs, concatenated, go through the output projection into the residual
stream (v10_triton_paged_gqa/layer/gqa.py:14-146; formulas
v00_full_recompute/layer/gqa.py:43-91).

All sizes are parameters: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias,
o_bias, window, scale, positions.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, POSITIONS, KVSpec, Mixer, TensorSpec, build_part
from .linear import Linear


@MIXERS.register("attention")
class AttentionMixer(Mixer):
    graph_safe = True  # nothing is planned on the host for single-token steps

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qkv_bias = bool(p.get("qkv_bias", True))
        self.o_bias = bool(p.get("o_bias", False))
        self.window: Optional[int] = p.get("window")
        scale = p.get("scale")
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        if self.head_dim % 8 or self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is not supported (multiples of 8 up to 256)")
        self.positions = build_part(POSITIONS, p["positions"]) if p.get("positions") else None
        # single-token steps are replayed from a CUDA graph only if the position encoding, too,
        # plans nothing on the host
        self.graph_safe = getattr(self.positions, "graph_safe", True)
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.qkv_proj: Linear | None = None
        self.o_proj: Linear | None = None

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.num_kv_heads, self.head_dim, self.window)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, d = int(p["hidden_size"]), int(p["head_dim"])
        q_size, kv_size = int(p["num_heads"]) * d, int(p["num_kv_heads"]) * d
        out = []
        for name, rows in (("q_proj", q_size), ("k_proj", kv_size), ("v_proj", kv_size)):
            out.append(TensorSpec(f"{prefix}{name}.weight", (rows, hidden)))
            if p.get("qkv_bias", True):
                out.append(TensorSpec(f"{prefix}{name}.bias", (rows,)))
        out.append(TensorSpec(f"{prefix}o_proj.weight", (hidden, q_size)))
        if p.get("o_bias", False):
            out.append(TensorSpec(f"{prefix}o_proj.bias", (hidden,)))
        if p.get("positions"):  # a position encoding may have tensors of its own
            out += POSITIONS.get(p["positions"].kind).expected_tensors(p["positions"], prefix)
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        names = ("q_proj", "k_proj", "v_proj")
        weight = torch.cat([tensors[f"{prefix}{n}.weight"] for n in names], dim=0)
        bias = torch.cat([tensors[f"{prefix}{n}.bias"].float() for n in names], dim=0) if self.qkv_bias else None
        self.qkv_proj = Linear(weight, bias, device, dtype)
        self.o_proj = Linear(tensors[f"{prefix}o_proj.weight"],
                             tensors[f"{prefix}o_proj.bias"] if self.o_bias else None, device, dtype)
        if self.positions is not None:
            self.positions.load(tensors, prefix, device, dtype)

    def forward(self, ctx, x, acc, cache) -> None:
        tokens = x.shape[0]
        qkv = ctx.buffer("attention.qkv", (tokens, self.q_size + 2 * self.kv_size), ctx.dtype)
        positions = self.positions
        partials = self.qkv_proj.deferred(ctx, x) if getattr(positions, "accepts_partials", False) else None
        if partials is not None:
            positions.encode_and_store(ctx, qkv, self.num_heads, self.num_kv_heads, cache,
                                       partials=(partials[0], partials[1], self.qkv_proj.bias))
        else:
            self.qkv_proj.forward(x, qkv)
            if positions is not None and positions.stores_kv:
                positions.encode_and_store(ctx, qkv, self.num_heads, self.num_kv_heads, cache)
            else:  # no encoding at all, or one that only encodes: the mixer stores k and v itself
                if positions is not None:
                    positions.encode(ctx, qkv, self.num_heads, self.num_kv_heads)
                if cache.writable:
                    ops.store_kv(qkv, ctx.positions, ctx.token_req, cache.block_table, cache.pages, self.num_heads,
                                 self.num_kv_heads, self.head_dim, cache.page_size)
        out = ctx.buffer("attention.out", (tokens, self.q_size), ctx.dtype)
        from . import attention_bf16

        if not (ctx.dtype == torch.bfloat16 and attention_bf16.forward(self, ctx, qkv, cache, out)):
            ops.attention_generic(qkv, qkv.stride(0), cache.pages, cache.block_table, ctx.token_req,
                                  ctx.positions, out, tokens, self.num_heads, self.num_kv_heads,
                                  self.head_dim, cache.page_size, self.window, self.scale)
        if not self.o_proj.accumulate_later(ctx, out, acc):
            self.o_proj.forward(out, acc, accumulate=True)
