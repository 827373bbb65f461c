"""Sampling options and the rule that turns logits into a token.

The reference samples with ``logits.argmax`` only (v10_triton_paged_gqa/engine.py:187-188)
and stops a request on a stop id or after ``max_new_tokens`` (default 128,
v10_triton_paged_gqa/request.py:20, scheduler.py:255-266).  Temperature sampling is
added: a draw from softmax(logits / temperature) in float32 by the Gumbel-max rule
with a counter-based generator keyed by (seed, tokens sampled so far, vocabulary
index), so a request's draws do not depend on the batch it runs in.  The kernel is
``csrc/sampling.cu``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    max_new_tokens: int = 128
    temperature: float = 0.0  # 0: greedy (argmax, lowest index wins a tie)
    seed: Optional[int] = None  # None: derived from the request's arrival number
    stop_token_ids: tuple = ()
    ignore_eos: bool = False  # keep generating through stop ids (benchmarks)

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        self.stop_token_ids = tuple(int(t) for t in self.stop_token_ids)


@dataclass
class SampleSpec:
    """How to sample one row of a step: the request's temperature, seed and counter."""

    temperature: float = 0.0
    seed: int = 0
    counter: int = 0


__all__ = ["SamplingParams", "SampleSpec"]
