"""Device memory of the cache: one tensor of pages per group, one tensor of state rows
per layer execution that keeps fixed-size state.

Pages of a group: ``[layers in group, num_pages, 2 (k, v), kv_heads, page_size, head_dim]``
in the compute dtype, so that a page id means the same page in every layer of the group
(the reference's single tensor ``[2, L, blocks, kv_heads, block, d]`` has the same
property, v10_triton_paged_gqa/kvcache.py:19-28) and one (page, kv head) tile of keys is
a contiguous ``page_size x head_dim`` box.  Pages are never cleared when they change
hands: kernels read only positions the block table and the request's length cover.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .manager import CacheError, CacheManager, GroupSpec


@dataclass
class LayerCache:
    """What a mixer sees of the cache for one execution in one step."""

    pages: Optional[torch.Tensor]  # [num_pages, 2, kv_heads, page_size, head_dim]
    block_table: Optional[torch.Tensor]  # [requests in step, width] int32
    page_size: int
    state: Optional[torch.Tensor]  # [max_slots, *state shape]
    writable: bool
    group: int = -1


def plan_groups(needs: list, num_pages: int) -> tuple[list[GroupSpec], dict]:
    """Group the executions that own paged history by (kv_heads, head_dim, window).
    Returns the groups and a map entry -> (group index, layer index inside the group)."""
    keys, members = [], {}
    for need in needs:
        if need.kv is None or need.owner != need.entry:
            continue
        key = need.kv.group_key()
        if key not in members:
            keys.append(key)
            members[key] = []
        members[key].append(need.entry)
    groups, where = [], {}
    for g, key in enumerate(keys):
        groups.append(GroupSpec(key[0], key[1], key[2], tuple(members[key]), num_pages))
        for i, entry in enumerate(members[key]):
            where[entry] = (g, i)
    return groups, where


class CacheStorage:
    def __init__(self, needs: list, page_size: int, max_slots: int, num_pages: int, max_seq_len: int,
                 device, dtype: torch.dtype):
        self.needs = needs
        self.page_size = page_size
        self.groups, self.where = plan_groups(needs, num_pages)
        element = torch.empty((), dtype=dtype).element_size()
        need = sum(len(g.entries) * g.num_pages * 2 * g.num_kv_heads * page_size * g.head_dim * element for g in self.groups)
        if torch.device(device).type == "cuda":
            free, _ = torch.cuda.mem_get_info(device)
            if need > free:
                raise CacheError(
                    f"the page pool needs {need / 2**30:.1f} GiB ({num_pages} pages of {page_size} tokens for "
                    f"{max_slots} slots), {free / 2**30:.1f} GiB are free: lower max_num_blocks, max_seq_len or "
                    "max_decode_slots")
        self.manager = CacheManager(self.groups, page_size, max_slots, max_seq_len)
        self.pages = [
            torch.zeros((len(g.entries), g.num_pages, 2, g.num_kv_heads, page_size, g.head_dim), device=device, dtype=dtype)
            for g in self.groups
        ]
        self.states = {}
        for need in needs:
            if need.state is not None:
                self.states[need.entry] = torch.zeros((max_slots, *need.state.shape), device=device,
                                                      dtype=getattr(torch, need.state.dtype))

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.pages) + sum(
            t.numel() * t.element_size() for t in self.states.values())

    def clear_slot(self, slot: int) -> None:
        """Zero the state rows of a slot (at admission)."""
        for state in self.states.values():
            state[slot].zero_()

    def layer_caches(self, block_tables: list) -> list[LayerCache]:
        """The per-execution view for one step; ``block_tables[g]`` is group g's table."""
        out = []
        for need in self.needs:
            pages = table = None
            group = -1
            if need.kv is not None:
                group, layer = self.where[need.owner]
                pages, table = self.pages[group][layer], block_tables[group]
            out.append(LayerCache(pages, table, self.page_size, self.states.get(need.entry),
                                  writable=need.owner == need.entry, group=group))
        return out
