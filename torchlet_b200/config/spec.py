"""Architecture-neutral description of a model: which parts, with which constants,
in which order.

A typed architecture configuration (for instance ``Qwen2Config``) is turned into a
``ModelSpec``; everything below the configuration layer (weights, parts, cache,
engine) reads only the ``ModelSpec``.  The reference passes the same constants as
constructor arguments layer by layer
(v10_triton_paged_gqa/layer/transformer_block.py:10-35); here they are data so that
layers may differ from one another and the run order is a list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its registered kind and its own constants."""

    kind: str
    params: dict = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class NormSlot:
    """One norm of a layer: the role the block arrangement knows it by (for instance
    "mixer_norm"), its part, and the tensor-name prefix of its weights below the layer's."""

    role: str
    part: PartSpec
    prefix: str


@dataclass(frozen=True)
class LayerSpec:
    """One layer's parts and where their tensors are found.

    ``prefix`` is the tensor-name prefix of the layer; each part's tensors lie below
    ``prefix + <part prefix>``.  The part prefixes are the checkpoint's own names, set by the
    architecture's configuration; nothing below the configuration layer spells one out.
    ``norms`` holds as many norms as the block arrangement ``block`` asks for, by role.
    """

    prefix: str
    block: str  # arrangement of the parts, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    norms: tuple = ()  # of NormSlot
    mixer_prefix: str = "mixer."
    feed_forward_prefix: str = "feed_forward."

    def norm(self, role: str) -> NormSlot:
        for slot in self.norms:
            if slot.role == role:
                return slot
        raise KeyError(f"layer {self.prefix!r} has no norm for the role {role!r}; "
                       f"it has: {', '.join(s.role for s in self.norms) or 'none'}")


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers`` and may appear more than once in the
    schedule.  Each entry owns the cache of its execution unless ``cache_from``
    names an earlier entry, whose cache it then reads without writing.
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    embedding_name: str
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    final_norm_prefix: str
    lm_head_name: str
    tie_word_embeddings: bool

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("the layer schedule is empty")
        for i, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(
                    f"schedule entry {i} names layer {entry.layer}, "
                    f"but there are {len(self.layers)} layers"
                )
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < i:
                    raise ValueError(
                        f"schedule entry {i} reads the cache of entry {entry.cache_from}, "
                        "which must be an earlier entry"
                    )
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(
                        f"schedule entry {i} reads the cache of entry {entry.cache_from}, "
                        "which owns no cache itself"
                    )
