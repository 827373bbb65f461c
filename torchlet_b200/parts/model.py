"""A model put together from a ``ModelSpec``: embedding, the layers run in the order
of the schedule, final norm, LM head (embedding -> blocks -> norm -> head,
v10_triton_paged_gqa/model/qwen2_5.py:21-87).  It knows no architecture by name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..config.spec import ModelSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, KVSpec, StateSpec, TensorSpec, build_part
from .linear import Linear


@dataclass
class ExecutionCacheNeed:
    """What one schedule entry keeps between steps."""

    entry: int
    owner: int  # the entry whose cache is used (itself unless cache_from is set)
    kv: Optional[KVSpec]
    state: Optional[StateSpec]


def _layer_parts(layer) -> list:
    """(registry, part description, full tensor-name prefix, role) of every part of a layer, in the
    order their tensors are listed and loaded.  The names come from the layer's description."""
    parts = [(NORMS, slot.part, layer.prefix + slot.prefix, slot.role) for slot in layer.norms]
    parts.insert(min(1, len(parts)), (MIXERS, layer.mixer, layer.prefix + layer.mixer_prefix, "mixer"))
    parts.append((FEED_FORWARDS, layer.feed_forward, layer.prefix + layer.feed_forward_prefix, "feed_forward"))
    return parts


def expected_tensors(spec: ModelSpec) -> list[TensorSpec]:
    """Every tensor the checkpoint must hold, by name, with its shape."""
    out = [TensorSpec(spec.embedding_name, (spec.vocab_size, spec.hidden_size))]
    for layer in spec.layers:
        for registry, part, prefix, _ in _layer_parts(layer):
            out += registry.get(part.kind).expected_tensors(part, prefix)
    out += NORMS.get(spec.final_norm.kind).expected_tensors(spec.final_norm, spec.final_norm_prefix)
    out.append(TensorSpec(spec.lm_head_name, (spec.vocab_size, spec.hidden_size), optional=spec.tie_word_embeddings))
    return out


class LayeredModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks = []
        for layer in spec.layers:
            block_cls = BLOCKS.get(layer.block)
            missing = [role for role in block_cls.norm_roles if role not in {slot.role for slot in layer.norms}]
            if missing:
                raise ValueError(f"layer {layer.prefix!r}: the arrangement {layer.block!r} needs norms for {missing}")
            self.blocks.append(
                block_cls(
                    build_part(MIXERS, layer.mixer),
                    build_part(FEED_FORWARDS, layer.feed_forward),
                    {slot.role: build_part(NORMS, slot.part) for slot in layer.norms},
                )
            )
        self.final_norm = build_part(NORMS, spec.final_norm)
        self.embedding: torch.Tensor | None = None
        self.lm_head: Linear | None = None
        self.dtype: torch.dtype | None = None
        self.device = None

    # ------------------------------------------------------------ structure
    def cache_needs(self) -> list[ExecutionCacheNeed]:
        needs = []
        for i, entry in enumerate(self.spec.schedule):
            mixer = self.blocks[entry.layer].mixer
            owner = i if entry.cache_from is None else entry.cache_from
            if entry.cache_from is not None:
                theirs = self.blocks[self.spec.schedule[owner].layer].mixer.kv_spec()
                mine = mixer.kv_spec()
                if theirs is None or mine is None or (theirs.num_kv_heads, theirs.head_dim) != (mine.num_kv_heads, mine.head_dim):
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {owner}: shapes differ")
            needs.append(ExecutionCacheNeed(i, owner, mixer.kv_spec(), mixer.state_spec()))
        return needs

    # --------------------------------------------------------------- weights
    def load(self, tensors: dict, device, dtype: torch.dtype) -> None:
        """Lay the checkpoint's tensors (by name) out on the device for the kernels."""
        spec = self.spec
        self.device, self.dtype = torch.device(device), dtype
        self.embedding = tensors[spec.embedding_name].to(device=device, dtype=dtype).contiguous()
        for layer, block in zip(spec.layers, self.blocks):
            for _, _, prefix, role in _layer_parts(layer):
                part = {"mixer": block.mixer, "feed_forward": block.feed_forward}.get(role) or block.norms[role]
                part.load(tensors, prefix, device, dtype)
        self.final_norm.load(tensors, spec.final_norm_prefix, device, dtype)
        if spec.tie_word_embeddings:
            self.lm_head = Linear.from_device_weight(self.embedding)
        else:
            self.lm_head = Linear(tensors[spec.lm_head_name], None, device, dtype)

    # --------------------------------------------------------------- forward
    def forward(self, ctx, caches: list) -> torch.Tensor:
        """Run the step's tokens through the schedule; returns the float32 stream [T, hidden]."""
        acc = ctx.buffer("stream", (ctx.num_tokens, self.spec.hidden_size), torch.float32)
        ops.embed(self.embedding, ctx.tokens, acc)
        for i, entry in enumerate(self.spec.schedule):
            self.blocks[entry.layer].forward(ctx, acc, caches[i])
        ctx.flush_pending()
        return acc

    def logits(self, ctx, acc: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        """Float32 logits of the stream rows ``rows`` (int32) into ``out`` [len(rows), vocab]."""
        x = self.final_norm.apply(ctx, acc, rows=rows, name="final.normed")
        self.lm_head.forward(x, out)
