"""Engine options.

The reference's engine takes ``max_decode_slots=4, kv_block_size=16,
max_num_blocks=None`` (v10_triton_paged_gqa/engine.py:22-47): the width of the
decode batch, tokens per page, and the pool size including the reserved page 0.
Those names and meanings are kept; the token budget and the dtype are added.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"  # "bfloat16" (serving kernels) or "float32" (true 32-bit)
    max_decode_slots: int = 4  # most requests live at a time
    kv_block_size: int = 16  # tokens per page
    max_num_blocks: Optional[int] = None  # pool size incl. reserved page 0; None: never runs out
    max_seq_len: Optional[int] = None  # None: max_position_embeddings
    max_num_batched_tokens: int = 2048  # token budget of one step
    cuda_graph: bool = True  # capture decode-only steps
    # a waiting request is admitted beside running ones only if the pools have pages for all its tokens
    # and this many for every running request to grow into (None: on the pages of its first portion)
    admission_headroom: Optional[int] = 1
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        aliases = {"bf16": "bfloat16", "fp32": "float32", "bfloat16": "bfloat16", "float32": "float32"}
        if self.dtype not in aliases:
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        self.dtype = aliases[self.dtype]
        if self.max_decode_slots <= 0:
            raise ValueError("max_decode_slots must be positive")
        if self.kv_block_size <= 0:
            raise ValueError("kv_block_size must be positive")
        if self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_batched_tokens must be positive")
        if self.max_num_blocks is not None and self.max_num_blocks < 2:
            raise ValueError("max_num_blocks must be at least 2 (page 0 is reserved)")

    def resolve(self, max_position_embeddings: int) -> "EngineConfig":
        """Fill the defaults that depend on the model."""
        if self.max_seq_len is None:
            self.max_seq_len = max_position_embeddings
        if self.max_seq_len > max_position_embeddings:
            raise ValueError(
                f"max_seq_len {self.max_seq_len} exceeds max_position_embeddings "
                f"{max_position_embeddings}"
            )
        if self.max_num_blocks is None:
            # as the reference: enough for every slot at full length, plus page 0
            self.max_num_blocks = self.max_decode_slots * ceil_div(self.max_seq_len, self.kv_block_size) + 1
        return self
